// Fused GGUF prefill GEMM ("umma" variant) on tcgen05 tensor cores with TMEM accumulators, M >= 9.
//
// C[M,N] = A[M,K] * dequant(W[N,K])^T (+ bias), float16 / bfloat16; all nine weight types (Q8_0, Q4_0, Q2_K .. Q6_K, MXFP4, NVFP4)
// (the kernel template lives in this header; umma_gemm_<type>.cu instantiates it per weight type).
// Tensor-core bound for M >= 512 (Q6_K 4096x14336: 1248 FLOP per weight byte at M = 512).
//
// Swap-AB: the weight tile is the UMMA "A" operand (128 rows = UMMA M), the activation tile is "B"
// (BM rows = UMMA N, 64..256), so D[n, m] lives in TMEM as 128 lanes x BM fp32 columns and one CTA
// reuses every dequantized weight tile across BM activation rows.  The weight operand is fed from TENSOR MEMORY
// (tcgen05.mma with A in TMEM): a 128 x 64 bf16 tile is 128 lanes x 32 columns, four such slots sit behind the
// accumulator columns, so the dequantized weights never touch shared memory - at 128 x 256 x 16 per instruction
// the MMA's shared-memory reads alone would otherwise take 3/4 of the SM's shared-memory bandwidth.  Per CTA:
//   * warp 18, one lane: TMA of the PACKED bytes of 128 weight rows x one 256-weight super-block (a 2-D byte
//     tensor map over the weight, box = 128 rows x the 16-byte aligned window around the block) into a
//     3-deep shared-memory ring.  One instruction per 18-30 KB: no thread spends issue slots on the copy.
//   * 16 producer warps (512 threads): wait for the packed super-block, copy their own words to registers,
//     release the ring slot, then unpack.  Warps 0-7 produce the two 64-wide K stages of the first
//     half of the super-block, warps 8-15 those of the second half; thread (row = 32*(warp%4)+lane,
//     half = (warp%8)/4) unpacks 32 weights per stage with 32-bit logic + packed bf16x2/f16x2 math and
//     writes them to its TMEM lane with two tcgen05.st.32x32b.x8 (16 columns of 2 x 16-bit);
//     tcgen05.wait::st + mbarrier arrive.  The two groups only meet at mbarriers, never at a CTA barrier.
//   * warp 16, one lane: TMA (cp.async.bulk.tensor.2d, SWIZZLE_128B, no multicast) of the BM x 64
//     activation tile per stage; rows past M are zero-filled by the tensor map.
//   * warp 17, one lane: tcgen05.mma.cta_group::1.kind::f16 (128 x BM x 16, four per stage), then
//     tcgen05.commit onto the stage's "empty" barrier; after the last stage onto the accumulator barrier.
//   * epilogue: the 16 producer warps read TMEM (tcgen05.ld 32x32b.x16; warp%4 picks the lane quarter,
//     warp/4 the column quarter), add bias, convert and store.
// Work split is stream-K: one CTA per SM, each with the same number of (tile, super-block) units, so the tensor cores
// of every SM are busy for the whole launch whatever (M/BM)*(N/128) is.  A tile whose K range is cut between CTAs is
// finished by the CTA that holds its end: the others leave fp32 partial tiles in a library-owned workspace and raise a
// flag, the finisher adds them in a fixed order (see Walk below).  No second kernel, bit-reproducible results.
// The packed-weight tensor map needs weight rows that are multiples of 16 bytes: any K % 256 == 0 for the types whose 256
// weights take a multiple of 16 bytes, K % 512 == 0 for MXFP4 (136 bytes), K % 1024 == 0 for Q2_K (84), K % 2048 == 0 for
// Q6_K (210) and Q3_K (110).  Other
// shapes are served by the other variants.
//
// Every mbarrier wait is bounded: after kSpinLimit polls the waiter records a code in a device status
// word, raises a CTA-wide abort flag and every role falls through to the common teardown (outstanding
// TMA copies are waited for, TMEM is freed).  Nothing traps or spins forever.
//
// The reference has no counterpart kernel: its CUDA path dequantizes the whole weight to a dense
// scratch and calls an Sm80 mma.sync CUTLASS GEMM (src/dinoml/lowering/ops/gemm.py:729-749,
// kernels/cuda/src/cutlass_gemm.cu:56-89); the tile-level dequantize-then-MMA idea follows its
// prototype WMMA kernels (kernels/rocm/src/ck_gguf_q8_gemm.hip:1209-1618).
#pragma once
#include <cuda.h>

#include "gemv_mma_common.cuh"

namespace b200gguf {

int check_gemm_args(const void* a, const void* b, const void* c, int qtype, int dtype, int m, int n, int k);

namespace umma {

constexpr int kRowsW = 128;            // weight rows per CTA (UMMA M)
constexpr int kBK = 64;                // K per pipeline stage (one 128-byte swizzle atom of 16-bit values)
constexpr int kProducerThreads = 512;
constexpr int kGroupThreads = 256;     // producers of one K stage
constexpr int kThreads = kProducerThreads + 96;   // + activation TMA warp, MMA warp, packed-weight TMA warp
constexpr uint32_t kSpinLimit = 1u << 24;   // try_wait polls before a wait gives up (each poll suspends ~tens of ns or more)

enum : int { ST_OK = 0, ST_EMPTY_TIMEOUT = 1, ST_FULL_TIMEOUT = 2, ST_ACC_TIMEOUT = 3, ST_PEER_TIMEOUT = 4 };
constexpr uint32_t kFlagSpinLimit = 1u << 22;   // polls (200 ns apart) of another CTA's partial-tile flag

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (after flagging) if the phase never completes or the CTA is aborting.
// The non-blocking test comes first: on the MMA-issuing warp most waits find their phase already complete, and
// there test_wait measured ~90 cycles less than a try_wait that succeeds at once.
// Only one lane per warp polls (18 pollers per CTA), so there is no sleep back-off: try_wait itself suspends the
// thread for a hardware-defined slice.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (mbar_test_wait(bar, parity)) return true;
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  atomicCAS(status, 0, code);
  return false;
}
// The same wait made by a whole converged warp, with one answer for all lanes.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, status, code) ? 1 : 0) != 0;
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}\n" : "=r"(pred));
  return pred != 0;
}
// Bounded wait with no flagging, for teardown paths.
__device__ __forceinline__ void mbar_wait_plain(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return;
    if (i > 64) __nanosleep(40);
  }
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// K-major, SWIZZLE_128B shared-memory matrix descriptor: rows of 128 B, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return uint64_t((addr & 0x3ffffu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) |
         (uint64_t(2) << 61);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};\n" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
               "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
// A operand from tensor memory, B from shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 16-bit pair arithmetic used to turn quants into MMA operand values.
template <typename T> struct Pair;
template <> struct Pair<__nv_bfloat16> {
  static constexpr uint32_t kMagicBytes = 0x43434343u;   // 0x43qq = 128 + q
  static constexpr float kMagic = 128.f;
  static constexpr uint32_t kFormat = 1;                  // UMMA F16F32Format::BF16
  static constexpr int kFp4MagPos = 6;                    // FP4 codes: exponent / mantissa bits land on bits 6..8
  static constexpr float kFp4Up = 0x1p120f, kFp4Rest = 0x1p6f;   // bits = e2m1 * 2^-126; * kFp4Up is a normal number
  static constexpr CUtensorMapDataType kTmaType = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  using V = __nv_bfloat162;
  static __device__ __forceinline__ V splat(float f) { return __float2bfloat162_rn(f); }
  static __device__ __forceinline__ V pack(float lo, float hi) { return __floats2bfloat162_rn(lo, hi); }
  static __device__ __forceinline__ __nv_bfloat16 cvt(float f) { return __float2bfloat16_rn(f); }
  static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
};
template <> struct Pair<__half> {
  static constexpr uint32_t kMagicBytes = 0x64646464u;   // 0x64qq = 1024 + q
  static constexpr float kMagic = 1024.f;
  static constexpr uint32_t kFormat = 0;                  // UMMA F16F32Format::F16
  static constexpr int kFp4MagPos = 9;                    // bits 9..11
  static constexpr float kFp4Up = 0x1p14f, kFp4Rest = 1.f;       // bits = e2m1 * 2^-14
  static constexpr CUtensorMapDataType kTmaType = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  using V = __half2;
  static __device__ __forceinline__ V splat(float f) { return __float2half2_rn(f); }
  static __device__ __forceinline__ V pack(float lo, float hi) { return __floats2half2_rn(lo, hi); }
  static __device__ __forceinline__ __half cvt(float f) { return __float2half_rn(f); }
  static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
};
template <typename V> __device__ __forceinline__ V as_pair(uint32_t r) { return *reinterpret_cast<V*>(&r); }
template <typename V> __device__ __forceinline__ uint32_t as_u32(V v) { return *reinterpret_cast<uint32_t*>(&v); }

// 4 quant bytes (values 0..255, here < 64) -> two pairs of (value - offset) * scale [+ addend].
template <typename T>
__device__ __forceinline__ void bytes_to_pairs(uint32_t u, typename Pair<T>::V off, typename Pair<T>::V scale, typename Pair<T>::V add,
                                               uint32_t& p01, uint32_t& p23) {
  using V = typename Pair<T>::V;
  const V a = __hsub2(as_pair<V>(__byte_perm(u, Pair<T>::kMagicBytes, 0x4140)), off);
  const V b = __hsub2(as_pair<V>(__byte_perm(u, Pair<T>::kMagicBytes, 0x4342)), off);
  p01 = as_u32<V>(__hfma2(a, scale, add));
  p23 = as_u32<V>(__hfma2(b, scale, add));
}

// 16 packed bytes starting S*2 bytes past a 16-byte aligned shared address, as four 32-bit words.  Q6_K
// blocks are only 2-byte aligned, so their fields sit at one of 8 byte phases inside the staged chunks;
// S is that phase (uniform across a warp whenever the weight rows are 16-byte multiples).
template <int S>
__device__ __forceinline__ void fetch16(const uint8_t* aligned, uint32_t* out) {
  const uint4 c0 = *reinterpret_cast<const uint4*>(aligned);
  if (S == 0) {
    out[0] = c0.x; out[1] = c0.y; out[2] = c0.z; out[3] = c0.w;
    return;
  }
  const uint4 c1 = *reinterpret_cast<const uint4*>(aligned + 16);
  const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  constexpr int j = S >> 1;
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = (S & 1) ? __funnelshift_r(w[j + i], w[j + i + 1], 16) : w[j + i];
}
template <int S>
__device__ __forceinline__ void q6k_fetch(const uint8_t* rowbase, int hb, int lhalf, uint32_t* qw, uint32_t* tail) {
  fetch16<S>(rowbase + 64 * hb + 16 * lhalf, qw);             // ql, quads 0/2
  fetch16<S>(rowbase + 64 * hb + 32 + 16 * lhalf, qw + 4);    // ql, quads 1/3
  fetch16<S>(rowbase + 128 + 32 * hb + 16 * lhalf, qw + 8);   // qh
  fetch16<S>(rowbase + 192, tail);                            // 16 int8 scales
  fetch16<S>(rowbase + 208, tail + 4);                        // d (first 2 bytes)
}

// Packed super-block window in shared memory: the 16-byte aligned span that contains one block of every row.
// Q4_K blocks (144 B) are always aligned; a Q6_K block (210 B) starts 0..14 bytes into its window and the last
// field read (d, through a 32-byte fetch at +208) ends at byte 240.  Eight Q8_0 blocks (272 B per 256 weights, always
// 16-byte aligned) are wider than a TMA box may be (256 elements), so they travel as two boxes of 144 B: blocks 0..3
// start at byte 0 of the first, blocks 4..7 at byte 8 of the second (which starts at byte 128 of the 272).  Every pitch
// is an odd number of 16-byte chunks, so 16-byte reads of 8 consecutive rows hit all 32 banks.
//   kSuper: packed bytes per 256 weights of a row; kBoxes: TMA boxes per super-block; kSlots: super-blocks in the ring.
template <int QT> struct RawGeom;
template <> struct RawGeom<QTYPE_Q4_K> { static constexpr int kPitch = 144, kSuper = 144, kBoxes = 1, kSlots = 3; };
template <> struct RawGeom<QTYPE_Q5_K> { static constexpr int kPitch = 176, kSuper = 176, kBoxes = 1, kSlots = 3; };   // Q4_K + 32 bytes of fifth bits
template <> struct RawGeom<QTYPE_Q6_K> { static constexpr int kPitch = 240, kSuper = 210, kBoxes = 1, kSlots = 3; };
template <> struct RawGeom<QTYPE_Q8_0> { static constexpr int kPitch = 144, kSuper = 272, kBoxes = 2, kSlots = 2; };
template <> struct RawGeom<QTYPE_Q4_0> { static constexpr int kPitch = 144, kSuper = 144, kBoxes = 1, kSlots = 3; };   // 8 blocks of 18 B
template <> struct RawGeom<QTYPE_MXFP4> { static constexpr int kPitch = 144, kSuper = 136, kBoxes = 1, kSlots = 3; };  // 8 x 17 B, starts 0 / 8 bytes into its window
template <> struct RawGeom<QTYPE_Q2_K> { static constexpr int kPitch = 112, kSuper = 84, kBoxes = 1, kSlots = 3; };    // starts 0 / 4 / 8 / 12 bytes into its window
template <> struct RawGeom<QTYPE_Q3_K> { static constexpr int kPitch = 144, kSuper = 110, kBoxes = 1, kSlots = 3; };   // any even phase, like Q6_K
template <> struct RawGeom<QTYPE_NVFP4> { static constexpr int kPitch = 144, kSuper = 144, kBoxes = 1, kSlots = 3; };  // 4 blocks of 36 B

// One Q8_0 block (B = 0..7 inside the 256 weights) of a row: 16 of its int8 quants (half LHALF) and its scale.
// win: this row inside the box that holds blocks 4*(B/4) .. 4*(B/4)+3.
template <int B>
__device__ __forceinline__ void q8_fetch(const uint8_t* win, int lhalf, uint32_t* qw, float& d) {
  constexpr int kStart = 8 * (B >> 2) + 34 * (B & 3);      // block start inside its box
  constexpr int kPhase = ((kStart + 2) & 15) >> 1;
  fetch16<kPhase>(win + ((kStart + 2) & ~15) + 16 * lhalf, qw);
  d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(win + kStart));
}
// 4 int8 quants -> two 16-bit pairs of q * d, each rounded once.  With u = q + 128 in byte 1 of a float's mantissa,
// f = 2^23 + 256 u, and f * (d / 256) - (2^23 + 2^15) * (d / 256) = q * d with every term exact in fp32.
template <typename T>
__device__ __forceinline__ void q8_to_pairs(uint32_t u, float d256, float c, uint32_t& p01, uint32_t& p23) {
  using P = Pair<T>;
  const uint32_t v = u ^ 0x80808080u;
  const float f0 = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7404));
  const float f1 = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7414));
  const float f2 = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7424));
  const float f3 = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7434));
  p01 = as_u32<typename P::V>(P::pack(fmaf(f0, d256, c), fmaf(f1, d256, c)));
  p23 = as_u32<typename P::V>(P::pack(fmaf(f2, d256, c), fmaf(f3, d256, c)));
}

// ---- Q2_K (scales[16], qs[64], d, dmin: 84 B) and Q3_K (hmask[32], qs[64], scales[12], d: 110 B).  Weight 128*hb + 32*j + l of a
// super-block is bits 2j, 2j+1 of qs[32*hb + l] (Q3_K: plus bit 4*hb + j of hmask[l] as a third bit, less 4); its scale index is
// 8*hb + 2*j + l/16.  Thread (hb, h16) of a row takes the 16 qs bytes l = 16*h16 .. +15 of half-block hb: all four j of them.
template <int S>
__device__ __forceinline__ void q2k_fetch(const uint8_t* rowbase, int hb, int h16, uint32_t* qw, uint32_t* scw, uint32_t* tail) {
  fetch16<S>(rowbase + 16 + 32 * hb + 16 * h16, qw);
  fetch16<S>(rowbase, scw);            // 16 bytes: 4-bit scale | 4-bit min << 4 per sub-block
  fetch16<S>(rowbase + 80, tail);      // d, dmin in the first word
}
template <int S>
__device__ __forceinline__ void q3k_fetch(const uint8_t* rowbase, int hb, int h16, uint32_t* qw, uint32_t* scw) {
  fetch16<S>(rowbase + 32 + 32 * hb + 16 * h16, qw);
  fetch16<S>(rowbase + 16 * h16, qw + 4);     // the third bits of weights l = 16*h16 .. +15, one bit position per (hb, j)
  fetch16<S>(rowbase + 96, scw);              // 12 scale bytes, then d
}

// ---- the 4-bit types with 32-weight blocks (Q4_0: u16 d + 16 bytes of nibbles, 18 B; MXFP4: u8 e + the same, 17 B).
// Byte j of a block holds weight j (low nibble) and weight j + 16 (high nibble), so the two threads of a row split a
// block by BYTES: thread half lh takes bytes 8*lh .. 8*lh+7, i.e. weights 8*lh .. +7 and 16 + 8*lh .. +7 (four TMEM
// columns each).  The four blocks of half a super-block start R0 bytes past the 16-byte aligned address `base`; blocks
// are only 1- or 2-byte aligned, so the words are rebuilt from aligned 16-byte loads with funnel shifts whose amounts
// are compile-time constants (R0 is one of four values, chosen by a switch at the call site).
//   qw[2b], qw[2b+1]: the 8 bytes of block b; sc[b]: the word whose low bits are the block's scale field.
template <int R0, int BB, int QOFF>
__device__ __forceinline__ void blk32_fetch(const uint8_t* base, int lh, uint32_t* qw, uint32_t* sc) {
  uint32_t w[21];
#pragma unroll
  for (int c = 0; c < 5; ++c) {
    const uint4 v = *reinterpret_cast<const uint4*>(base + 16 * c);
    w[4 * c] = v.x; w[4 * c + 1] = v.y; w[4 * c + 2] = v.z; w[4 * c + 3] = v.w;
  }
  w[20] = 0;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int o = R0 + BB * b + QOFF, i0 = o >> 2, sh = 8 * (o & 3);
    const uint32_t a0 = lh ? w[i0 + 2] : w[i0], a1 = lh ? w[i0 + 3] : w[i0 + 1], a2 = lh ? w[i0 + 4] : w[i0 + 2];
    qw[2 * b] = sh ? __funnelshift_r(a0, a1, sh) : a0;
    qw[2 * b + 1] = sh ? __funnelshift_r(a1, a2, sh) : a1;
    const int oe = R0 + BB * b;
    sc[b] = w[oe >> 2] >> (8 * (oe & 3));
  }
}
// FP4 (e2m1) codes -> 16-bit operand values, exactly.  A code s|ee|m placed on the sign bit, the two lowest exponent
// bits and the top mantissa bit of a 16-bit float IS that format's own number e2m1 * 2^(1 - bias): its subnormals give
// the codes 0 and 0.5.  Two exact multiplies follow: by k1 (which lifts the value into the normal range) and by the
// block scale.  e2m1 has 2 significant bits, an e8m0 scale none and a ue4m3 scale 4: the product is exact in either
// 16-bit type while it stays in range.  w = 4 bytes; lo / hi = the values of their low / high nibbles as two pairs.
template <typename T>
__device__ __forceinline__ void fp4_to_pairs(uint32_t w, typename Pair<T>::V k1, typename Pair<T>::V scale, uint32_t* lo, uint32_t* hi) {
  using P = Pair<T>;
  using V = typename P::V;
  constexpr uint32_t kMag = (7u << P::kFp4MagPos) * 0x00010001u;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const uint32_t t = __byte_perm(w, 0u, j == 0 ? 0x1404u : 0x3424u);   // bytes 2j, 2j+1 on bits 8..15 / 24..31
    // low nibble: sign on bit 11, magnitude on bits 8..10; high nibble: sign on bit 15, magnitude on bits 12..14
    uint32_t lmag;
    if constexpr (P::kFp4MagPos >= 8) lmag = t << (P::kFp4MagPos - 8); else lmag = t >> (8 - P::kFp4MagPos);
    const uint32_t l = ((t << 4) & 0x80008000u) | (lmag & kMag);
    const uint32_t h = (t & 0x80008000u) | ((t >> (12 - P::kFp4MagPos)) & kMag);
    lo[j] = as_u32<V>(__hmul2(__hmul2(as_pair<V>(l), k1), scale));
    hi[j] = as_u32<V>(__hmul2(__hmul2(as_pair<V>(h), k1), scale));
  }
}
// ue4m3 scale byte (NVFP4) times `mult`, where mult carries 2^120: the byte placed on exponent / mantissa bits of a float
// is value * 2^-120 (fp32 subnormals give the ue4m3 subnormals).  0x7f decodes to 0 as in the reference's host code.
__device__ __forceinline__ float ue4m3_times(uint32_t x, float mult) {
  x &= 0xffu;
  return x == 0x7fu ? 0.f : __fmul_rn(__uint_as_float((x & 0x7fu) << 20), mult);
}

// Rings.  A super-block (256 weights of every row) is kStagesPerSb = 4 K stages; a stage is a weight-tile slot in TMEM (32
// columns, right after the BM accumulator columns) paired with an activation tile in shared memory.
//   BM = 256: the ring is one super-block of stages, each with its own full / empty barrier pair - the MMAs of one stage
//     (512 tensor cycles) are longer than the barrier handling on the issuing warp, fine-grained hand-over keeps the
//     tensor pipe fed.
//   BM <= 128: the MMAs of a stage are shorter than one wait + commit on the issuing warp (~300 cycles), which then paces
//     the whole CTA.  There the hand-over is per SUPER-BLOCK (one wait, 16 MMAs, one commit) and the ring is
//     stage_units<BM>() super-blocks deep, so that the round trip commit -> empty -> tcgen05.st -> full is hidden.
// Packed ring: raw_slots<QT, BM>() super-blocks of packed bytes in shared memory (TMA), as many as fit up to 6 when the
// super-blocks are short-lived.
constexpr int kStagesPerSb = 4;         // 256 weights / kBK: the MMA loop relies on it
constexpr int kWSlotCols = kBK / 2;     // 64 16-bit values per lane = 32 columns
constexpr int kSmemBudget = 227 * 1024;
template <int BM> constexpr bool coarse_handover() { return BM < 256; }
template <int BM> constexpr int stage_units() { return BM >= 256 ? 1 : BM >= 128 ? 2 : 3; }
template <int BM> constexpr int x_tile_bytes() { return BM * kBK * 2; }
template <int QT> constexpr int raw_box_bytes() { return kRowsW * RawGeom<QT>::kPitch; }
template <int QT> constexpr int raw_slot_bytes() { return RawGeom<QT>::kBoxes * raw_box_bytes<QT>(); }
template <int BM> constexpr int tmem_cols() { return BM + stage_units<BM>() * kStagesPerSb * kWSlotCols > 256 ? 512 : 256; }
template <int QT, int BM> constexpr int raw_slots() {
  constexpr int fit = (kSmemBudget - 1024 - 512 - stage_units<BM>() * kStagesPerSb * x_tile_bytes<BM>()) / raw_slot_bytes<QT>();
  constexpr int want = BM >= 256 ? RawGeom<QT>::kSlots : 6;
  return fit < want ? fit : want;
}
template <int QT, int BM> constexpr size_t smem_bytes() {
  return 1024 + size_t(stage_units<BM>() * kStagesPerSb) * x_tile_bytes<BM>() + size_t(raw_slots<QT, BM>()) * raw_slot_bytes<QT>() + 512;
}

struct Params {
  const void* bias;       // [n] or null
  void* out;              // [m, n] in the activation dtype
  float* partial;         // one fp32 tile [BM][128] per CTA (stream-K partial sums)
  int* flags;             // one word per CTA: 1 = that CTA's partial tile is complete in `partial`
  int* status;            // device status word
  int m, n, k;
  int m_tiles;            // activation tiles per weight panel
  long long units;        // output tiles x super-blocks
  PeerOut peers;          // extra destinations of the output (SCATTER kernels only)
};

// Stream-K work split.  The work of the launch is a line of units (tile t, super-block sb), tile-major; CTA c of G owns
// the contiguous range [start(c), start(c+1)), so every SM gets the same amount of tensor-core work whatever the tile
// count.  A CTA walks its range from the HIGHEST tile down; the segment that holds the end of a tile is therefore the
// last thing its CTA does, and the other pieces of that tile belong to lower-numbered CTAs that computed them first.
// Those CTAs store an fp32 partial tile and raise a flag; the CTA with the end of the tile adds the partials in CTA
// order to its own accumulator, applies bias and stores (deterministic summation order).  Dependencies only point to
// lower-numbered CTAs, which are dispatched first, and every flag wait is bounded.
__device__ __forceinline__ long long unit_start(int c, long long units, int ctas) { return (static_cast<long long>(c) * units) / ctas; }
__device__ __forceinline__ int unit_owner(long long u, long long units, int ctas) { return int(((u + 1) * ctas - 1) / units); }

struct Walk {
  long long u0, u1;
  int nsb;
  __device__ __forceinline__ int tile_hi() const { return int((u1 - 1) / nsb); }
  __device__ __forceinline__ int tile_lo() const { return int(u0 / nsb); }
  __device__ __forceinline__ void segment(int t, int& sb_b, int& sb_e) const {
    const long long base = static_cast<long long>(t) * nsb;
    sb_b = int((u0 > base ? u0 : base) - base);
    sb_e = int((u1 < base + nsb ? u1 : base + nsb) - base);
  }
};

__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(int* p, int v) { asm volatile("st.release.gpu.global.s32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory"); }

// SCATTER: finished tiles are also stored to the extra destinations in p.peers (other GPUs' gather buffers).
template <int QT, typename T, int BM, bool SCATTER>
__global__ void __launch_bounds__(kThreads, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map, const Params p) {
  using P = Pair<T>;
  using V = typename P::V;
  constexpr bool COARSE = coarse_handover<BM>();
  constexpr int U = stage_units<BM>(), NS = U * kStagesPerSb, NSR = raw_slots<QT, BM>();    // stage ring (weight tile in TMEM + activation tile in smem), packed ring
  constexpr int NB = COARSE ? U : NS;          // full / empty barrier pairs: one per super-block slot or one per stage
  static_assert(COARSE || U == 1, "per-stage hand-over runs on a ring of one super-block");
  static_assert(NSR >= 2 && BM + NS * kWSlotCols <= 512 && (2 * NB + 2 * NSR + 4) * 8 + 8 <= 512, "rings");
  constexpr int kXTile = x_tile_bytes<BM>();
  constexpr uint32_t kTmemCols = tmem_cols<BM>();
  constexpr int kPitch = RawGeom<QT>::kPitch;
  constexpr int kRawBytes = raw_slot_bytes<QT>();
  constexpr int kBlockBytes = RawGeom<QT>::kSuper;
  constexpr uint32_t kIdesc = (1u << 4) | (P::kFormat << 7) | (P::kFormat << 10) | (uint32_t(BM >> 3) << 17) |
                              (uint32_t(kRowsW >> 4) << 24);
  constexpr uint32_t kWarpArrivals = kGroupThreads / 32;     // one elected arrive per producer warp of a group

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* xtiles = smem;                                              // NS x [BM][128 B]
  uint8_t* raw = xtiles + NS * kXTile;                                 // NSR x [128][kPitch]
  uint64_t* bars = reinterpret_cast<uint64_t*>(raw + NSR * kRawBytes);
  // bars: full[NB], empty[NB], rawfull[NSR], rawfree[NSR], accumulator full, accumulator free, drain, epilogue.  A stage is "full"
  // when its 8 producer warps have written the weight tile AND the activation tile's bytes have landed (one barrier, one
  // wait for the MMA warp); it is "empty" when the MMAs that read it have completed (one tcgen05.commit, watched by
  // producers and TMA).
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NB + 2 * NSR + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (NB + s); };
  auto rawfull = [&](int s) { return bar0 + 8u * (2 * NB + s); };
  auto rawfree = [&](int s) { return bar0 + 8u * (2 * NB + NSR + s); };
  const uint32_t accbar = bar0 + 8u * (2 * NB + 2 * NSR), accfree = accbar + 8u, drainbar = accbar + 16u, epibar = accbar + 24u;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x, ctas = gridDim.x;
  const int nsb = p.k >> 8;
  Walk walk;
  walk.u0 = unit_start(cta, p.units, ctas);
  walk.u1 = unit_start(cta + 1, p.units, ctas);
  walk.nsb = nsb;
  const bool has_work = walk.u1 > walk.u0;
  const int tile_hi = has_work ? walk.tile_hi() : -1, tile_lo = has_work ? walk.tile_lo() : 0;

  if (tid == 0) {
    for (int s = 0; s < NB; ++s) {
      mbar_init(full(s), (COARSE ? 2 : 1) * kWarpArrivals + 1);   // the producer warps that fill it + the TMA lane's arrive.expect_tx
      mbar_init(empty(s), 1);
    }
    for (int s = 0; s < NSR; ++s) {
      mbar_init(rawfull(s), 1);
      mbar_init(rawfree(s), kProducerThreads / 32);
    }
    mbar_init(accbar, 1);
    mbar_init(accfree, kProducerThreads / 32);
    mbar_init(drainbar, 1);
    mbar_init(epibar, kProducerThreads / 32);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 17) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch.  The next kernel in the stream may begin once every CTA of this grid is past this
  // point; its CTAs take over an SM as soon as one of ours exits.  In the other direction, the packed weights are
  // constants: the weight TMA, the unpack and the tcgen05.st of this grid run ahead of `griddepcontrol.wait`, which only
  // the activation TMA warp (before its first load) and the producers (before their first epilogue: outputs, partial
  // tiles and flags are shared with the preceding launch) execute.
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

  if (warp < 16) {
    // ------------------------------------------------------------------ producers
    const int grp = warp >> 3;                                  // which half of the super-block (two K stages)
    const int row = 32 * (warp & 3) + lane, lhalf = (warp >> 2) & 1;
    bool alive = true;
    const uint32_t tmem_lane = tmem_base + (uint32_t(32 * (warp & 3)) << 16) + uint32_t(BM);   // this warp's lanes, first A column
    int it = 0, segi = 0;                                       // super-blocks / segments done by this CTA so far
    uint32_t epi_phase = 0;
    // Barrier over the 16 producer warps on an mbarrier, so that it is bounded like every other wait (a plain bar.sync
    // would hang the warps that reached it if another warp had given up).
    auto producer_sync = [&]() -> bool {
      __syncwarp();
      int ok = 1;
      if (lane == 0) {
        mbar_arrive(epibar);
        ok = mbar_wait(epibar, epi_phase & 1u, abort_flag, p.status, ST_ACC_TIMEOUT) ? 1 : 0;
      }
      ++epi_phase;
      return __shfl_sync(0xffffffffu, ok, 0) != 0;
    };
    // Epilogue of one segment (tile t, super-blocks [sb_b, sb_e), the segi-th of this CTA).  false = a wait gave up.
    bool dep_waited = false;
    auto epilogue = [&](int t, int sb_b, int sb_e, int segi) -> bool {
      if (!dep_waited) {
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
        dep_waited = true;
      }
      {
        int ok = 1;
        if (lane == 0) ok = mbar_wait(accbar, uint32_t(segi) & 1u, abort_flag, p.status, ST_ACC_TIMEOUT) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) return false;
      }
      tcgen05_fence_after();
      const int n0 = (t / p.m_tiles) * kRowsW, m0 = (t % p.m_tiles) * BM;
      const int n_row = n0 + row;
      const bool whole = sb_b == 0 && sb_e == nsb;
      const bool finishes = sb_e == nsb;            // this CTA stores the tile (after adding the others' partial sums)
      int peer0 = cta;                              // first CTA with a piece of this tile; peers are peer0 .. cta-1
      if (finishes && !whole) {
        peer0 = unit_owner(static_cast<long long>(t) * nsb, p.units, ctas);
        if (tid < cta - peer0) {
          bool seen = false;
          for (uint32_t i = 0; i < kFlagSpinLimit && !seen; ++i) {
            seen = ld_acquire(p.flags + peer0 + tid) != 0;
            if (!seen) __nanosleep(200);
          }
          if (!seen) { *abort_flag = 1; atomicCAS(p.status, 0, ST_PEER_TIMEOUT); }
        }
        if (!producer_sync()) return false;
      }
      const float bias_v = (finishes && p.bias != nullptr && n_row < p.n) ? P::up(static_cast<const T*>(p.bias)[n_row]) : 0.f;
      constexpr int kColsPerWarp = BM / 4;
      constexpr int CH = kColsPerWarp >= 32 ? 32 : 16;   // columns per round: enough independent loads / stores in flight
#pragma unroll
      for (int c0 = 0; c0 < kColsPerWarp; c0 += CH) {
        const int col = (warp >> 2) * kColsPerWarp + c0;
        uint32_t r[CH];
#pragma unroll
        for (int q = 0; q < CH / 16; ++q)
          tmem_ld16(tmem_base + (uint32_t(32 * (warp & 3)) << 16) + uint32_t(col + 16 * q), *reinterpret_cast<uint32_t(*)[16]>(&r[16 * q]));
        tmem_ld_wait();
        if (!finishes) {
          float* dst = p.partial + (static_cast<size_t>(cta) * BM + col) * kRowsW + row;     // tile-local [BM][128]
#pragma unroll
          for (int j = 0; j < CH; ++j) dst[j * kRowsW] = __uint_as_float(r[j]);
        } else {
          for (int peer = peer0; peer < cta; ++peer) {
            const float* src = p.partial + (static_cast<size_t>(peer) * BM + col) * kRowsW + row;
            float v[CH];
#pragma unroll
            for (int j = 0; j < CH; ++j) v[j] = __ldcg(src + j * kRowsW);
#pragma unroll
            for (int j = 0; j < CH; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + v[j]);
          }
          if (p.peers.act != ACT_NONE) {
            // gated pair: within every 16 weight rows the first 8 belong to the first matrix, the next 8 to the second;
            // lane l and lane l ^ 8 hold the two halves, the output has n / 2 columns
            const int out_row = ((n_row >> 4) << 3) + (n_row & 7);
            const int64_t n_out = p.n >> 1;
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const float mine = __uint_as_float(r[j]) + bias_v;       // bias interleaved like the rows (0 without one)
              const float other = __shfl_xor_sync(0xffffffffu, mine, 8);
              if ((lane & 8) == 0 && n_row < p.n && m0 + col + j < p.m) {
                const T v = P::cvt(gate_activation(mine, p.peers.act) * other);
                const int64_t at = int64_t(m0 + col + j) * n_out + out_row;
                static_cast<T*>(p.out)[at] = v;
                if (SCATTER) {
#pragma unroll
                  for (int pi = 0; pi < 8; ++pi)
                    if (pi < p.peers.count) static_cast<T*>(p.peers.ptr[pi])[at] = v;
                }
              }
            }
          } else if (n_row < p.n) {
            T* dst = static_cast<T*>(p.out) + int64_t(m0 + col) * p.n + n_row;
#pragma unroll
            for (int j = 0; j < CH; ++j)
              if (m0 + col + j < p.m) {
                const T v = P::cvt(__uint_as_float(r[j]) + bias_v);
                dst[int64_t(j) * p.n] = v;
                if (SCATTER) {
#pragma unroll
                  for (int pi = 0; pi < 8; ++pi)
                    if (pi < p.peers.count) static_cast<T*>(p.peers.ptr[pi])[int64_t(m0 + col + j) * p.n + n_row] = v;
                }
              }
          }
        }
      }
      if (!finishes) {
        // every producer thread's partial sums happen before the barrier; the release below is cumulative over them
        if (!producer_sync()) return false;
        if (tid == 0) { __threadfence(); st_release(p.flags + cta, 1); }
      } else if (!whole) {
        if (!producer_sync()) return false;    // every thread has read the peers' tiles
        if (tid < cta - peer0) p.flags[peer0 + tid] = 0;   // leave the flags clear for the next launch
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(accfree);             // the accumulator columns may be overwritten
      return true;
    };
    int pend_t = -1, pend_b = 0, pend_e = 0;                    // segment whose epilogue has not run yet
    for (int t = tile_hi; t >= tile_lo && alive; --t, ++segi) {
      int sb_b, sb_e;
      walk.segment(t, sb_b, sb_e);
      for (int sb = sb_b; sb < sb_e && alive; ++sb, ++it) {
        const int rslot = it % NSR;
        {
          int ok = 1;
          if (lane == 0) ok = mbar_wait(rawfull(rslot), uint32_t(it / NSR) & 1u, abort_flag, p.status, ST_FULL_TIMEOUT) ? 1 : 0;
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) { alive = false; break; }
        }
        const uint8_t* rowbase = raw + rslot * kRawBytes + row * kPitch;
        // ---- copy this thread's packed words to registers
        uint32_t qw[(QT == QTYPE_Q8_0 || QT == QTYPE_Q5_K) ? 16 : 12];
        float dscale = 0.f, dmin = 0.f;
        float sub_scale[4];                   // Q6_K: int8 scales of quads 0..3; Q8_0: d of this thread's four blocks
        float sub_min[4] = {0.f, 0.f, 0.f, 0.f};   // Q2_K: -dmin * min of the thread's four sub-blocks
        if constexpr (QT == QTYPE_Q8_0) {
          // blocks 4*grp .. 4*grp+3 sit in box grp of the slot; block 2*ls + h feeds half h of stage 2*grp + ls
          const uint8_t* win = rowbase + grp * raw_box_bytes<QT>();
          if (grp == 0) {
            q8_fetch<0>(win, lhalf, qw, sub_scale[0]);
            q8_fetch<1>(win, lhalf, qw + 4, sub_scale[1]);
            q8_fetch<2>(win, lhalf, qw + 8, sub_scale[2]);
            q8_fetch<3>(win, lhalf, qw + 12, sub_scale[3]);
          } else {
            q8_fetch<4>(win, lhalf, qw, sub_scale[0]);
            q8_fetch<5>(win, lhalf, qw + 4, sub_scale[1]);
            q8_fetch<6>(win, lhalf, qw + 8, sub_scale[2]);
            q8_fetch<7>(win, lhalf, qw + 12, sub_scale[3]);
          }
        } else if constexpr (QT == QTYPE_Q4_K || QT == QTYPE_Q5_K) {
          constexpr int kQsOff = QT == QTYPE_Q5_K ? 48 : 16;      // Q5_K keeps 32 bytes of fifth bits between the scales and the nibbles
          const uint4 hdr = *reinterpret_cast<const uint4*>(rowbase);
          dscale = half_bits_to_float(uint16_t(hdr.x & 0xffffu));
          dmin = half_bits_to_float(uint16_t(hdr.x >> 16));
          // sub-blocks 4*grp .. 4*grp+3 belong to this thread's two stages
          const uint32_t scw = grp == 0 ? (hdr.y & 0x3f3f3f3fu) : ((hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4));
          const uint32_t mnw = grp == 0 ? (hdr.z & 0x3f3f3f3fu) : (((hdr.w >> 4) & 0x0f0f0f0fu) | (((hdr.z >> 6) & 0x03030303u) << 4));
          qw[8] = scw;
          qw[9] = mnw;
#pragma unroll
          for (int ls = 0; ls < 2; ++ls) {
            const uint4 q = *reinterpret_cast<const uint4*>(rowbase + kQsOff + 64 * grp + 32 * ls + 16 * lhalf);
            qw[4 * ls] = q.x; qw[4 * ls + 1] = q.y; qw[4 * ls + 2] = q.z; qw[4 * ls + 3] = q.w;
          }
          if constexpr (QT == QTYPE_Q5_K) {     // bit 2*(2*grp+ls) + {0, 1} of qh byte l: fifth bit of weight l in the low / high sub-block
            const uint4 qh = *reinterpret_cast<const uint4*>(rowbase + 16 + 16 * lhalf);
            qw[12] = qh.x; qw[13] = qh.y; qw[14] = qh.z; qw[15] = qh.w;
          }
          sub_scale[0] = sub_scale[1] = sub_scale[2] = sub_scale[3] = 0.f;
        } else if constexpr (QT == QTYPE_Q4_0 || QT == QTYPE_MXFP4) {
          constexpr int BB = QT == QTYPE_Q4_0 ? 18 : 17;
          // this thread's four blocks (4*grp ..) start a0 bytes into the row's window; block b feeds half b%2 of stage 2*grp + b/2
          const int a0 = ((sb * kBlockBytes) & 15) + 4 * BB * grp;
          const uint8_t* base = rowbase + (a0 & ~15);
          uint32_t scw[4];
          switch (a0 & 15) {
            case 0: blk32_fetch<0, BB, BB - 16>(base, lhalf, qw, scw); break;
            case 4: blk32_fetch<4, BB, BB - 16>(base, lhalf, qw, scw); break;
            case 8: blk32_fetch<8, BB, BB - 16>(base, lhalf, qw, scw); break;
            default: blk32_fetch<12, BB, BB - 16>(base, lhalf, qw, scw); break;
          }
#pragma unroll
          for (int b = 0; b < 4; ++b)
            sub_scale[b] = QT == QTYPE_Q4_0 ? half_bits_to_float(uint16_t(scw[b] & 0xffffu))
                                            : __fmul_rn(e8m0_half(scw[b] & 0xffu), 2.f * P::kFp4Rest);    // 2^(e - 127), less what k1 already gave
        } else if constexpr (QT == QTYPE_Q2_K) {
          uint32_t scw[4], tail[4];
          switch (((sb * kBlockBytes) & 15) >> 2) {        // 84-byte blocks: the phase inside the window is a multiple of 4
            case 0: q2k_fetch<0>(rowbase, grp, lhalf, qw, scw, tail); break;
            case 1: q2k_fetch<2>(rowbase, grp, lhalf, qw, scw, tail); break;
            case 2: q2k_fetch<4>(rowbase, grp, lhalf, qw, scw, tail); break;
            default: q2k_fetch<6>(rowbase, grp, lhalf, qw, scw, tail); break;
          }
          dscale = half_bits_to_float(uint16_t(tail[0] & 0xffffu));
          dmin = half_bits_to_float(uint16_t(tail[0] >> 16));
#pragma unroll
          for (int j = 0; j < 4; ++j) {       // scale byte 8*grp + 2*j + lhalf
            const uint32_t b = ((grp ? scw[2 + (j >> 1)] : scw[j >> 1]) >> (8 * (2 * (j & 1) + lhalf))) & 0xffu;
            sub_scale[j] = dscale * float(b & 0x0fu);
            sub_min[j] = -(dmin * float(b >> 4));
          }
        } else if constexpr (QT == QTYPE_Q3_K) {
          uint32_t scw[4];
          switch (((sb * kBlockBytes) & 15) >> 1) {
            case 0: q3k_fetch<0>(rowbase, grp, lhalf, qw, scw); break;
            case 1: q3k_fetch<1>(rowbase, grp, lhalf, qw, scw); break;
            case 2: q3k_fetch<2>(rowbase, grp, lhalf, qw, scw); break;
            case 3: q3k_fetch<3>(rowbase, grp, lhalf, qw, scw); break;
            case 4: q3k_fetch<4>(rowbase, grp, lhalf, qw, scw); break;
            case 5: q3k_fetch<5>(rowbase, grp, lhalf, qw, scw); break;
            case 6: q3k_fetch<6>(rowbase, grp, lhalf, qw, scw); break;
            default: q3k_fetch<7>(rowbase, grp, lhalf, qw, scw); break;
          }
          dscale = half_bits_to_float(uint16_t(scw[3] & 0xffffu));
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // 6-bit scale number is = 8*grp + 2*j + lhalf = 4*q + i4: low nibble in byte (is % 8) (its high half for is >= 8), the two
            // high bits in byte 8 + i4 at bit 2*q
            const int i4 = 2 * (j & 1) + lhalf, q = 2 * grp + (j >> 1);
            const uint32_t low = (scw[j >> 1] >> (8 * i4 + 4 * grp)) & 0x0fu;
            const uint32_t high = (scw[2] >> (8 * i4 + 2 * q)) & 0x03u;
            sub_scale[j] = dscale * float(int(low | (high << 4)) - 32);
          }
        } else if constexpr (QT == QTYPE_NVFP4) {
          // stage 2*grp + ls is block 2*grp + ls (four ue4m3 scales, 32 bytes of nibbles); sub-blocks 2*lhalf and 2*lhalf + 1
          // (bytes 16*lhalf .. +15: weights 32*lhalf .. +31 of the stage) are this thread's
          if (grp == 0) {
            fetch16<2>(rowbase + 16 * lhalf, qw);
            fetch16<4>(rowbase + 32 + 16 * lhalf, qw + 4);
          } else {
            fetch16<6>(rowbase + 64 + 16 * lhalf, qw);
            fetch16<0>(rowbase + 112 + 16 * lhalf, qw + 4);
          }
#pragma unroll
          for (int ls = 0; ls < 2; ++ls) {
            const uint32_t dw = *reinterpret_cast<const uint32_t*>(rowbase + 36 * (2 * grp + ls)) >> (16 * lhalf);
            sub_scale[2 * ls] = ue4m3_times(dw, 0x1p120f * P::kFp4Rest);
            sub_scale[2 * ls + 1] = ue4m3_times(dw >> 8, 0x1p120f * P::kFp4Rest);
          }
        } else {
          const int hb = grp;
          uint32_t tail[8];                     // bytes 192..223 of the block: 16 int8 scales, then d
          // rows are 16-byte multiples, so the block's phase inside its window is the same for every row
          switch (((sb * kBlockBytes) & 15) >> 1) {
            case 0: q6k_fetch<0>(rowbase, hb, lhalf, qw, tail); break;
            case 1: q6k_fetch<1>(rowbase, hb, lhalf, qw, tail); break;
            case 2: q6k_fetch<2>(rowbase, hb, lhalf, qw, tail); break;
            case 3: q6k_fetch<3>(rowbase, hb, lhalf, qw, tail); break;
            case 4: q6k_fetch<4>(rowbase, hb, lhalf, qw, tail); break;
            case 5: q6k_fetch<5>(rowbase, hb, lhalf, qw, tail); break;
            case 6: q6k_fetch<6>(rowbase, hb, lhalf, qw, tail); break;
            default: q6k_fetch<7>(rowbase, hb, lhalf, qw, tail); break;
          }
          dscale = half_bits_to_float(uint16_t(tail[4] & 0xffffu));
          // scale byte of quad i: 8*hb + 2*i + lhalf -> word 2*hb + i/2, byte 2*(i%2) + lhalf
          const uint32_t sw0 = hb ? tail[2] : tail[0], sw1 = hb ? tail[3] : tail[1];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t wsel = i < 2 ? sw0 : sw1;
            sub_scale[i] = float(int(int8_t(wsel >> (8 * (2 * (i & 1) + lhalf)))));
          }
        }
        __syncwarp();                          // every lane holds its words: the ring slot may be refilled
        if (lane == 0) mbar_arrive(rawfree(rslot));
        // K stage ls (0 / 1) of this thread's half of the super-block -> two groups of 8 words: 16 values each for
        // k' = 16*lhalf .. +15 and k' = 32 + 16*lhalf .. +15 of the 64-wide stage.
        auto unpack_stage = [&](int ls, uint32_t (&o0)[8], uint32_t (&o1)[8]) {
          if constexpr (QT == QTYPE_Q8_0) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const float d256 = sub_scale[2 * ls + h] * (1.f / 256.f);
              const float c = -8421376.f * d256;        // -(2^23 + 2^15) * d / 256, exact
              uint32_t (&o)[8] = h == 0 ? o0 : o1;
#pragma unroll
              for (int i = 0; i < 4; ++i) q8_to_pairs<T>(qw[8 * ls + 4 * h + i], d256, c, o[2 * i], o[2 * i + 1]);
            }
          } else if constexpr (QT == QTYPE_Q4_K || QT == QTYPE_Q5_K) {
            // stage = 64-weight group: low nibbles -> its first sub-block (k' 0..31), high nibbles -> its second (k' 32..63)
            const int sh = 16 * ls;
            const float sc0 = float((qw[8] >> sh) & 0xff), sc1 = float((qw[8] >> (sh + 8)) & 0xff);
            const float mn0 = float((qw[9] >> sh) & 0xff), mn1 = float((qw[9] >> (sh + 8)) & 0xff);
            const V off = P::splat(P::kMagic);
            const V s_lo = P::splat(dscale * sc0), a_lo = P::splat(-(dmin * mn0));
            const V s_hi = P::splat(dscale * sc1), a_hi = P::splat(-(dmin * mn1));
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t lo = qw[4 * ls + i] & 0x0f0f0f0fu, hi = (qw[4 * ls + i] >> 4) & 0x0f0f0f0fu;
              if constexpr (QT == QTYPE_Q5_K) {
                const int j = 2 * (2 * grp + ls);
                lo |= ((qw[12 + i] >> j) & 0x01010101u) * 16u;
                hi |= ((qw[12 + i] >> (j + 1)) & 0x01010101u) * 16u;
              }
              bytes_to_pairs<T>(lo, off, s_lo, a_lo, o0[2 * i], o0[2 * i + 1]);
              bytes_to_pairs<T>(hi, off, s_hi, a_hi, o1[2 * i], o1[2 * i + 1]);
            }
          } else if constexpr (QT == QTYPE_Q2_K || QT == QTYPE_Q3_K) {
            // stage 2*grp + ls = (half-block grp, j = 2*ls and 2*ls + 1): both halves come from the same 16 bytes at bit 2j
            const V off = P::splat(P::kMagic + (QT == QTYPE_Q3_K ? 4.f : 0.f));
#pragma unroll
            for (int qo = 0; qo < 2; ++qo) {
              const int j = 2 * ls + qo;
              uint32_t (&o)[8] = qo == 0 ? o0 : o1;
              const V s2 = P::splat(sub_scale[j]), a2 = P::splat(sub_min[j]);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint32_t nq = (qw[i] >> (2 * j)) & 0x03030303u;
                if constexpr (QT == QTYPE_Q3_K) nq |= ((qw[4 + i] >> (4 * grp + j)) & 0x01010101u) << 2;
                bytes_to_pairs<T>(nq, off, s2, a2, o[2 * i], o[2 * i + 1]);
              }
            }
          } else if constexpr (QT == QTYPE_Q4_0) {
            // o0 / o1 = blocks 2*ls, 2*ls+1 of this thread's four: [0..3] the low nibbles (weights 8*lhalf .. +7 of the block),
            // [4..7] the high nibbles (weights 16 + 8*lhalf .. +7)
            const V off = P::splat(P::kMagic + 8.f), zero = P::splat(0.f);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t (&o)[8] = h == 0 ? o0 : o1;
              const V d2 = P::splat(sub_scale[2 * ls + h]);
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                const uint32_t w = qw[2 * (2 * ls + h) + i];
                bytes_to_pairs<T>(w & 0x0f0f0f0fu, off, d2, zero, o[2 * i], o[2 * i + 1]);
                bytes_to_pairs<T>((w >> 4) & 0x0f0f0f0fu, off, d2, zero, o[4 + 2 * i], o[4 + 2 * i + 1]);
              }
            }
          } else if constexpr (QT == QTYPE_MXFP4) {
            const V k1 = P::splat(P::kFp4Up);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t (&o)[8] = h == 0 ? o0 : o1;
              const V sc2 = P::splat(sub_scale[2 * ls + h]);
#pragma unroll
              for (int i = 0; i < 2; ++i) fp4_to_pairs<T>(qw[2 * (2 * ls + h) + i], k1, sc2, &o[2 * i], &o[4 + 2 * i]);
            }
          } else if constexpr (QT == QTYPE_NVFP4) {
            // o0 / o1 = sub-blocks 2*lhalf, 2*lhalf+1 of the stage's block: 8 bytes each, low nibbles = its first 8 weights
            const V k1 = P::splat(P::kFp4Up);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t (&o)[8] = h == 0 ? o0 : o1;
              const V sc2 = P::splat(sub_scale[2 * ls + h]);
#pragma unroll
              for (int i = 0; i < 2; ++i) fp4_to_pairs<T>(qw[4 * ls + 2 * h + i], k1, sc2, &o[2 * i], &o[4 + 2 * i]);
            }
          } else {
            // stage = (half block grp, quad pair ls): quads 2*ls (k' 0..31) and 2*ls+1 (k' 32..63)
            const V off = P::splat(P::kMagic + 32.f);
            const V zero = P::splat(0.f);
#pragma unroll
            for (int qo = 0; qo < 2; ++qo) {
              const int quad = 2 * ls + qo;
              const V s2 = P::splat(dscale * sub_scale[quad]);
              uint32_t (&o)[8] = qo == 0 ? o0 : o1;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const uint32_t l4 = (qw[4 * qo + i] >> (4 * ls)) & 0x0f0f0f0fu;
                // the two high bits of quad q sit at bit 2q of the qh byte; they belong at bit 4
                const uint32_t hs = quad == 0 ? qw[8 + i] << 4 : quad == 1 ? qw[8 + i] << 2 : quad == 2 ? qw[8 + i] : qw[8 + i] >> 2;
                bytes_to_pairs<T>(l4 | (hs & 0x30303030u), off, s2, zero, o[2 * i], o[2 * i + 1]);
              }
            }
          }
        };
        // Where a stage's 2 x 16 values go in this thread's TMEM lane (a column = two 16-bit values): by default K values
        // 16*lhalf .. +15 and 32 + 16*lhalf .. +15; the byte-split types write four runs of 8; NVFP4 one run of 32.
        auto store_stage = [&](uint32_t tile, const uint32_t (&o0)[8], const uint32_t (&o1)[8]) {
          if constexpr (QT == QTYPE_Q4_0 || QT == QTYPE_MXFP4) {
            tmem_st4(tile + 4 * lhalf, o0);
            tmem_st4(tile + 8 + 4 * lhalf, o0 + 4);
            tmem_st4(tile + 16 + 4 * lhalf, o1);
            tmem_st4(tile + 24 + 4 * lhalf, o1 + 4);
          } else if constexpr (QT == QTYPE_NVFP4) {
            tmem_st8(tile + 16 * lhalf, o0);
            tmem_st8(tile + 16 * lhalf + 8, o1);
          } else {
            tmem_st8(tile + 8 * lhalf, o0);
            tmem_st8(tile + 16 + 8 * lhalf, o1);
          }
        };
        // one lane polls the barrier, the warp follows
        auto wait_empty = [&](int b, int trip) -> bool {
          int ok = 1;
          if (lane == 0) ok = mbar_wait(empty(b), uint32_t(trip - 1) & 1u, abort_flag, p.status, ST_EMPTY_TIMEOUT) ? 1 : 0;
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (ok) tcgen05_fence_after();
          return ok != 0;
        };
        if constexpr (COARSE) {
          // hand-over per super-block: unpack both stages (no TMEM slot needed yet), then wait for the slot, store, signal once
          const int ub = it % U, trip = it / U;
          uint32_t ow[2][2][8];
          unpack_stage(0, ow[0][0], ow[0][1]);
          unpack_stage(1, ow[1][0], ow[1][1]);
          if (trip > 0 && !wait_empty(ub, trip)) { alive = false; break; }
#pragma unroll
          for (int ls = 0; ls < 2; ++ls) {
            const uint32_t tile = tmem_lane + uint32_t((ub * kStagesPerSb + 2 * grp + ls) * kWSlotCols);
            store_stage(tile, ow[ls][0], ow[ls][1]);
          }
          tmem_st_wait();
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(full(ub));
        } else {
#pragma unroll
          for (int ls = 0; ls < 2; ++ls) {
            const int slot = 2 * grp + ls;       // stage ring slot = K stage inside the super-block
            if (it > 0 && !wait_empty(slot, it)) { alive = false; break; }
            const uint32_t tile = tmem_lane + uint32_t(slot * kWSlotCols);   // column k'/2 of this slot
            uint32_t o0[8], o1[8];
            unpack_stage(ls, o0, o1);
            store_stage(tile, o0, o1);
            tmem_st_wait();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(full(slot));
          }
        }
        if (!alive) break;
        // The previous segment's epilogue runs only now, after the first super-block of this segment has been unpacked:
        // the MMA warp finds its next weight tiles ready the moment the accumulator is handed back.
        if (sb == sb_b && pend_t >= 0) {
          if (!epilogue(pend_t, pend_b, pend_e, segi - 1)) { alive = false; break; }
          pend_t = -1;
        }
      }
      if (!alive) break;
      pend_t = t; pend_b = sb_b; pend_e = sb_e;
    }
    if (alive && pend_t >= 0) epilogue(pend_t, pend_b, pend_e, segi - 1);
  } else if (warp == 16) {
    // ------------------------------------------------------------------ activation TMA
    asm volatile("griddepcontrol.wait;\n" ::: "memory");     // the activations may be the preceding kernel's output
    // The three control warps stay converged: every lane runs the loop and polls the barriers, one elected lane issues
    // the asynchronous instructions.  Inside a divergent `if (lane == 0)` region the compiler cannot keep descriptors,
    // coordinates and barrier addresses in uniform registers, and each tcgen05.mma / bulk copy then costs tens of cycles
    // of register shuffling on the one thread the whole pipeline waits for.
    int it = 0;
    bool ok = true;
    for (int t = tile_hi; t >= tile_lo && ok; --t) {
      int sb_b, sb_e;
      walk.segment(t, sb_b, sb_e);
      const int m0 = (t % p.m_tiles) * BM;
      for (int sb = sb_b; sb < sb_e && ok; ++sb, ++it) {
        if constexpr (COARSE) {
          const int ub = it % U, trip = it / U;
          if (trip > 0 && !warp_wait(empty(ub), uint32_t(trip - 1) & 1u, abort_flag, p.status, ST_EMPTY_TIMEOUT)) { ok = false; break; }
          if (elect_one()) {
            mbar_arrive_expect_tx(full(ub), uint32_t(kStagesPerSb * kXTile));
#pragma unroll
            for (int st = 0; st < kStagesPerSb; ++st)
              tma_load_2d(smem_u32(xtiles + (ub * kStagesPerSb + st) * kXTile), &x_map, full(ub), sb * 256 + st * kBK, m0);
          }
          __syncwarp();
        } else {
#pragma unroll
          for (int slot = 0; slot < NS; ++slot) {
            if (it > 0 && !warp_wait(empty(slot), uint32_t(it - 1) & 1u, abort_flag, p.status, ST_EMPTY_TIMEOUT)) { ok = false; break; }
            if (elect_one()) {
              mbar_arrive_expect_tx(full(slot), uint32_t(kXTile));
              tma_load_2d(smem_u32(xtiles + slot * kXTile), &x_map, full(slot), sb * 256 + slot * kBK, m0);
            }
            __syncwarp();
          }
        }
      }
    }
    // Aborting: up to NS activation copies may still be writing shared memory, and their barrier also counts producer
    // arrivals that will never come, so it cannot be waited on.  A copy of this size lands within microseconds; give
    // the last ones a millisecond before the CTA may exit.
    if (*abort_flag)
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  } else if (warp == 18) {
    // ------------------------------------------------------------------ packed-weight TMA
    int it = 0;
    bool ok = true;
    for (int t = tile_hi; t >= tile_lo && ok; --t) {
      int sb_b, sb_e;
      walk.segment(t, sb_b, sb_e);
      const int n0 = (t / p.m_tiles) * kRowsW;
      for (int sb = sb_b; sb < sb_e; ++sb, ++it) {
        const int slot = it % NSR, use = it / NSR;
        if (use > 0 && !warp_wait(rawfree(slot), uint32_t(use - 1) & 1u, abort_flag, p.status, ST_EMPTY_TIMEOUT)) { ok = false; break; }
        if (elect_one()) {
          mbar_arrive_expect_tx(rawfull(slot), uint32_t(kRawBytes));
          // x coordinate = block start rounded down to 16 bytes; rows past N and bytes past the row end read as zero
          tma_load_2d(smem_u32(raw + slot * kRawBytes), &w_map, rawfull(slot), (sb * kBlockBytes) & ~15, n0);
          if constexpr (RawGeom<QT>::kBoxes == 2)     // second half of the super-block: blocks 4..7 start 8 bytes in
            tma_load_2d(smem_u32(raw + slot * kRawBytes + raw_box_bytes<QT>()), &w_map, rawfull(slot), sb * kBlockBytes + 128, n0);
        }
        __syncwarp();
      }
    }
    if (*abort_flag) {
      for (int i = max(0, it - NSR); i < it; ++i) mbar_wait_plain(rawfull(i % NSR), uint32_t(i / NSR) & 1u);
    }
  } else {
    // ------------------------------------------------------------------ MMA issue
    bool ok = true;
    const uint64_t db0 = smem_desc_sw128(smem_u32(xtiles));
    int it = 0, segi = 0;
    for (int t = tile_hi; t >= tile_lo && ok; --t, ++segi) {
      int sb_b, sb_e;
      walk.segment(t, sb_b, sb_e);
      if (segi > 0) {                        // the previous segment's accumulator has been read out
        ok = warp_wait(accfree, uint32_t(segi - 1) & 1u, abort_flag, p.status, ST_ACC_TIMEOUT);
        if (!ok) break;
        tcgen05_fence_after();
      }
      for (int sb = sb_b; sb < sb_e && ok; ++sb, ++it) {
        if constexpr (COARSE) {
          // one wait, sixteen MMAs, one commit per super-block
          const int ub = it % U;
          ok = warp_wait(full(ub), uint32_t(it / U) & 1u, abort_flag, p.status, ST_FULL_TIMEOUT);
          if (!ok) break;
          tcgen05_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int st = 0; st < kStagesPerSb; ++st) {
              const int slot = ub * kStagesPerSb + st;
#pragma unroll
              for (int kk = 0; kk < kBK / 16; ++kk)
                umma_f16_ts(tmem_base, tmem_base + uint32_t(BM + slot * kWSlotCols + 8 * kk), db0 + uint64_t((slot * kXTile) >> 4) + uint64_t(2 * kk),
                            kIdesc, (sb > sb_b || st > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(empty(ub));
          }
          __syncwarp();
        } else {
          // one super-block = NS stages per trip: slot numbers, TMEM columns and descriptor offsets are compile-time constants
#pragma unroll
          for (int slot = 0; slot < NS; ++slot) {
            ok = warp_wait(full(slot), uint32_t(it) & 1u, abort_flag, p.status, ST_FULL_TIMEOUT);
            if (!ok) break;
            tcgen05_fence_after();
            if (elect_one()) {
#pragma unroll
              for (int kk = 0; kk < kBK / 16; ++kk)      // 16 K values = 8 TMEM columns of A, 32 bytes of each B row
                umma_f16_ts(tmem_base, tmem_base + uint32_t(BM + slot * kWSlotCols + 8 * kk), db0 + uint64_t((slot * kXTile) >> 4) + uint64_t(2 * kk),
                            kIdesc, (sb > sb_b || slot > 0 || kk > 0) ? 1u : 0u);
              umma_commit(empty(slot));
            }
            __syncwarp();
          }
        }
      }
      if (ok && elect_one()) umma_commit(accbar);
      __syncwarp();
    }
    if (!ok && has_work && elect_one()) {   // aborting: let every MMA already issued finish before TMEM is freed
      umma_commit(drainbar);
      mbar_wait_plain(drainbar, 0);
    }
    __syncwarp();
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 17) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------- host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess) return EncodeTiledFn(nullptr);
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

constexpr int kMaxCtas = 1024;      // flag words per device; the grid never exceeds the SM count

// Tile shape and stream-K grid of one problem.
struct Plan {
  int bm, m_tiles, ctas;
  long long units;
  size_t workspace_bytes;     // fp32 partial tiles, one per CTA; 0 when every CTA range ends on a tile boundary
};

// Where a launch finds its partial-tile workspace, flags and status word.
struct Scratch { float* workspace; int* flags; int* status; };

template <int QT, typename T, int BM>
int launch(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, const Plan& pl, Scratch sc,
                  const PeerOut& peers, cudaStream_t s) {
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr) return RC_LAUNCH;
  const cuuint32_t estr[2] = {1, 1};
  CUtensorMap x_map, w_map;
  {   // activations [m, k], 16-bit: box = one K stage x BM rows, 128-byte swizzle (the MMA's B operand layout)
    const cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(m)};
    const cuuint64_t strides[1] = {cuuint64_t(k) * 2};
    const cuuint32_t box[2] = {cuuint32_t(kBK), cuuint32_t(BM)};
    if (enc(&x_map, Pair<T>::kTmaType, 2, const_cast<void*>(a), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return RC_LAUNCH;
  }
  {   // packed weight as bytes [n, row_bytes]: box = the aligned window around one block x 128 rows, no swizzle
    const cuuint64_t row_bytes = cuuint64_t(k / 256) * RawGeom<QT>::kSuper;
    const cuuint64_t dims[2] = {row_bytes, cuuint64_t(n)};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {cuuint32_t(RawGeom<QT>::kPitch), cuuint32_t(kRowsW)};
    if (enc(&w_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(b), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return RC_LAUNCH;
  }
  const bool scatter = peers.count > 0;
  auto kern = scatter ? gemm_umma_kernel<QT, T, BM, true> : gemm_umma_kernel<QT, T, BM, false>;
  constexpr size_t smem = smem_bytes<QT, BM>();
  static_assert(smem <= size_t(kSmemBudget), "shared-memory rings exceed the per-CTA limit");
  // The opt-in beyond 48 KB of dynamic shared memory belongs to the current device: set on every launch (a cheap host
  // call), so that a process driving several GPUs is right on each of them.
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return RC_LAUNCH;
  Params p;
  p.bias = bias;
  p.out = c;
  p.partial = sc.workspace;
  p.flags = sc.flags;
  p.status = sc.status;
  p.m = m; p.n = n; p.k = k;
  p.m_tiles = pl.m_tiles;
  p.units = pl.units;
  p.peers = peers;
  // programmatic stream serialization: see the griddepcontrol notes in the kernel
  if (gemv_launch(kern, pl.ctas, 1, kThreads, smem, s, x_map, w_map, p) != cudaSuccess) return RC_LAUNCH;
  return cudaGetLastError() == cudaSuccess ? RC_OK : RC_LAUNCH;
}

// Every instantiation of one weight type: the activation dtype and the tile height are picked at run time.  One
// translation unit per weight type calls this (umma_gemm_<type>.cu), so the types compile in parallel.
template <int QT>
int launch_qtype(int dtype, const void* a, const void* b, const void* bias, void* c, int m, int n, int k, const Plan& pl, Scratch sc,
                 const PeerOut& peers, cudaStream_t s) {
  if (dtype == DINO_BF16) {
    switch (pl.bm) {
      case 64: return launch<QT, __nv_bfloat16, 64>(a, b, bias, c, m, n, k, pl, sc, peers, s);
      case 128: return launch<QT, __nv_bfloat16, 128>(a, b, bias, c, m, n, k, pl, sc, peers, s);
      default: return launch<QT, __nv_bfloat16, 256>(a, b, bias, c, m, n, k, pl, sc, peers, s);
    }
  }
  switch (pl.bm) {
    case 64: return launch<QT, __half, 64>(a, b, bias, c, m, n, k, pl, sc, peers, s);
    case 128: return launch<QT, __half, 128>(a, b, bias, c, m, n, k, pl, sc, peers, s);
    default: return launch<QT, __half, 256>(a, b, bias, c, m, n, k, pl, sc, peers, s);
  }
}

// One function per weight type, each defined in its own translation unit.
#define B200_UMMA_LAUNCH_ARGS                                                                                                   \
  int dtype, const void *a, const void *b, const void *bias, void *c, int m, int n, int k, const Plan &pl, Scratch sc,          \
      const PeerOut &peers, cudaStream_t s
int launch_q4_k(B200_UMMA_LAUNCH_ARGS);
int launch_q5_k(B200_UMMA_LAUNCH_ARGS);
int launch_q6_k(B200_UMMA_LAUNCH_ARGS);
int launch_q8_0(B200_UMMA_LAUNCH_ARGS);
int launch_q4_0(B200_UMMA_LAUNCH_ARGS);
int launch_mxfp4(B200_UMMA_LAUNCH_ARGS);
int launch_nvfp4(B200_UMMA_LAUNCH_ARGS);
int launch_q2_k(B200_UMMA_LAUNCH_ARGS);
int launch_q3_k(B200_UMMA_LAUNCH_ARGS);

}  // namespace umma
}  // namespace b200gguf
