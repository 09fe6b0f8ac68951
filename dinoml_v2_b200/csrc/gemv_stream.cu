// Persistent decode GEMV ("stream" variant), M = 1..8, float16 / bfloat16 activations, tensor cores: Q4_K, Q5_K, Q6_K, Q4_0, Q2_K,
// Q3_K, MXFP4 and NVFP4 weights.
//
// C[M,N] = A[M,K] * dequant(W[N,K])^T (+ bias), W streamed once from HBM as packed GGUF blocks (Q4_K 144 B, Q6_K 210 B per
// 256 weights; Q6_K needs K % 2048 == 0 so that every row piece starts on a 16-byte boundary, other K stay with the tile
// kernel).  Same exact-integer tensor-core arithmetic as the tile kernels in gemv_mma.cu / gemv_q6k_mma.cu (quants become 16-bit floats 128+q /
// 1024+q, mma.sync.m16n8k16 with fp32 accumulation, per-sub-block scales applied in fp32, the offsets folded against
// per-sub-block activation sums); what changes is how the bytes move and how the work is cut:
//   * grid = one CTA per SM (or two).  The work of a launch is a line of units (16-row tile t, K chunk of 8 super-blocks),
//     tile-major; CTA c owns the contiguous range [c * U / G, (c + 1) * U / G), so every CTA moves the same number of bytes
//     whatever the tile count (688 tiles on 296 CTAs would otherwise be 2 or 3 tiles each).  A CTA walks its range from
//     the highest unit down: a tile cut between two CTAs is the FIRST thing the lower-numbered CTA computes (it leaves
//     its partial sums, 16 x M floats, in a small global workspace and raises a flag) and the LAST thing the
//     higher-numbered one computes (it adds the partial, lowers the flag and stores) - no waiting in practice, the
//     dependency points to a lower-numbered CTA, which is dispatched first, and the summation order is fixed.  One
//     prologue (activation sums) per CTA instead of one per tile;
//   * one producer warp issues, per (tile, K chunk of 8 super-blocks), sixteen 1-D bulk copies (cp.async.bulk, one per
//     weight row, 1152 B each) into a ring of D shared-memory stages; a stage is "full" when its bytes have landed
//     (mbarrier transaction count) and "empty" when its 8 consumer warps have arrived.  The ring runs across tile
//     boundaries.  No thread spends issue slots on per-16-byte copies and no CTA barrier sits in the loop;
//   * NG groups of 8 consumer warps take the stages round-robin (warp w of a group unpacks super-block w of the chunk
//     for all 16 rows), accumulate over the chunks of a tile and hand their partial rows to the epilogue warp through
//     a double-buffered shared-memory area guarded by mbarriers; the epilogue warp adds the partials in a fixed order,
//     applies bias / the gated activation and stores (also to peer buffers for the sharded path);
//   * programmatic dependent launch: the producer starts streaming the (constant) weights at once, everything that
//     reads activations or writes outputs first waits for the preceding kernel (griddepcontrol.wait).  With the
//     one-CTA-per-SM grid and at most half of an SM's shared memory and registers per CTA, the next launch's CTAs sit
//     beside this launch's and fill their rings while this one finishes.
// Every wait (mbarriers, the partial-tile flag) is bounded; one that gives up records a code (11..15) in the library's
// status word, raises the CTA's abort flag, the producer waits for the copies it has in flight, and every role returns.
//
// Behavioural ancestor in the reference: the small-M kernels of the fused prototype
// (kernels/rocm/src/ck_gguf_q8_gemm.hip:1009-1166); the reference's CUDA path dequantizes the whole weight and runs a
// dense Sm80 GEMM instead (src/dinoml/lowering/ops/gemm.py:729-749).
#include <map>
#include <type_traits>

#include "gemv_q6k_common.cuh"
#include "gemv_stream_common.cuh"

namespace b200gguf {

int check_gemm_args(const void* a, const void* b, const void* c, int qtype, int dtype, int m, int n, int k);

namespace stream {

constexpr int kRows = 16;                       // weight rows per tile (one MMA M-tile)
constexpr int kKC = 8;                          // super-blocks per row per stage: one per consumer warp of a group
// Bytes per super-block and shared-memory row pitch of a stage.  Q4_K: 8 x 144 + 32 = 1184 B, so that the 8-byte reads of 4
// rows x 4 lanes (a half-warp) hit 32 distinct banks.  Q6_K: 8 x 210 = 1680 B is 16 (mod 128) by itself, which spreads the
// 4-byte reads of 8 rows x 4 lanes over all banks; a block starts 2 bytes off a word boundary in every odd super-block.
template <int QT> struct Geom;
template <> struct Geom<QTYPE_Q4_K> { static constexpr int kSbBytes = 144, kPitch = kKC * 144 + 32; };
template <> struct Geom<QTYPE_Q6_K> { static constexpr int kSbBytes = 210, kPitch = kKC * 210; };
// Q5_K = the Q4_K block with 32 more bytes (one high bit per weight) between the scales and the nibbles: same 8-byte reads,
// 8 x 176 + 32 = 1440 B is 32 (mod 128) like the Q4_K pitch.
template <> struct Geom<QTYPE_Q5_K> { static constexpr int kSbBytes = 176, kPitch = kKC * 176 + 32; };
// The further types: packed bytes per 256 weights of a row; the pitch is the stage piece rounded up to 128 B, plus 16 (4 words:
// the 4-byte reads of 8 rows x 4 lanes hit 32 distinct banks) and every row starts 16-byte aligned (bulk-copy destination).
template <int BYTES> struct PaddedGeom { static constexpr int kSbBytes = BYTES, kPitch = (kKC * BYTES + 127) / 128 * 128 + 16; };
template <> struct Geom<QTYPE_Q4_0> : PaddedGeom<8 * 18> {};
template <> struct Geom<QTYPE_Q2_K> : PaddedGeom<84> {};
template <> struct Geom<QTYPE_Q3_K> : PaddedGeom<110> {};
template <> struct Geom<QTYPE_MXFP4> : PaddedGeom<8 * 17> {};
template <> struct Geom<QTYPE_NVFP4> : PaddedGeom<4 * 36> {};
// Q4_0 and MXFP4 (32-weight blocks: a scale and 16 bytes of nibbles), NVFP4, Q2_K and Q3_K run on tensor cores like Q4_K.
template <int QT> constexpr bool is_blk32() { return QT == QTYPE_Q4_0 || QT == QTYPE_MXFP4; }
template <int QT> constexpr bool is_q23() { return QT == QTYPE_Q2_K || QT == QTYPE_Q3_K; }     // 2- / 3-bit quants, a scale per 16 weights

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {     // selector bit 3 of a nibble: replicate the byte's sign bit
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
// 16-bit pair times 16-bit pair (one rounding per element; exact for the FP4 value x block scale products it is used for).
template <typename T> __device__ __forceinline__ uint32_t mul_pair(uint32_t a, uint32_t b);
template <> __device__ __forceinline__ uint32_t mul_pair<__half>(uint32_t a, uint32_t b) {
  const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t mul_pair<__nv_bfloat16>(uint32_t a, uint32_t b) {
  const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <typename T> __device__ __forceinline__ uint32_t splat_pair(float f);
template <> __device__ __forceinline__ uint32_t splat_pair<__half>(float f) {
  const __half2 v = __float2half2_rn(f);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t splat_pair<__nv_bfloat16>(float f) {
  const __nv_bfloat162 v = __float2bfloat162_rn(f);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// Eight FP4 (e2m1) codes of one 32-bit word -> their exact values as 16-bit MMA operand pairs: lo01 / lo23 = the low nibbles of
// bytes (0, 1) / (2, 3), hi01 / hi23 = the high nibbles.  Magnitudes come from byte look-up tables held in two registers
// (prmt with the codes as selector), the sign bit is OR-ed in.  No offset, no rounding: every e2m1 value is a 16-bit float.
template <typename T>
__device__ __forceinline__ void fp4x8_operands(uint32_t w, uint32_t& lo01, uint32_t& lo23, uint32_t& hi01, uint32_t& hi23) {
  const uint32_t m = w & 0x77777777u, w4 = w << 4;
  // sign of [b0.lo, b0.hi, b1.lo, b1.hi] and of [b2.lo, b2.hi, b3.lo, b3.hi] on bit 7 of a byte each
  const uint32_t sa = prmt(w4, w, 0xD9C8u) & 0x80808080u, sb = prmt(w4, w, 0xFBEAu) & 0x80808080u;
  if constexpr (std::is_same<T, __half>::value) {
    // 0, .5, 1, 1.5, 2, 3, 4, 6 as fp16: high bytes 00 38 3C 3E 40 42 44 46, low bytes zero
    const uint32_t ha = prmt(0x3E3C3800u, 0x46444240u, m) | sa, hb = prmt(0x3E3C3800u, 0x46444240u, m >> 16) | sb;
    lo01 = prmt(ha, 0u, 0x2404u); hi01 = prmt(ha, 0u, 0x3414u);
    lo23 = prmt(hb, 0u, 0x2404u); hi23 = prmt(hb, 0u, 0x3414u);
  } else {
    // as bf16: 0000 3F00 3F80 3FC0 4000 4040 4080 40C0
    const uint32_t ha = prmt(0x3F3F3F00u, 0x40404040u, m) | sa, hb = prmt(0x3F3F3F00u, 0x40404040u, m >> 16) | sb;
    const uint32_t la = prmt(0xC0800000u, 0xC0804000u, m), lb = prmt(0xC0800000u, 0xC0804000u, m >> 16);
    lo01 = prmt(la, ha, 0x6240u); hi01 = prmt(la, ha, 0x7351u);
    lo23 = prmt(lb, hb, 0x6240u); hi23 = prmt(lb, hb, 0x7351u);
  }
}

constexpr int kGroupWarps = kKC;
constexpr int kBarBytes = 256;                  // mbarrier area in front of the ring (up to 32 barriers)

static __device__ int g_stream_status;

template <int MXC, int NCW> struct RedBuf {
  float red[NCW][kRows][MXC];    // per consumer warp: sum_j ds * S' for (row, activation column)
  float xt[NCW][kRows][MXC];     // per consumer warp: sum_j (MAGIC * ds + dm) * X
};

template <int QT, int MXC, int NG, int D> constexpr size_t smem_fixed_bytes() {
  return kBarBytes /* barriers */ + size_t(D) * kRows * Geom<QT>::kPitch + 2 * sizeof(RedBuf<MXC, NG * kGroupWarps>);
}

// MXC: activation rows covered (power of two >= m, <= 8).  NG: groups of 8 consumer warps.  D: ring slots (D % NG == 0).
// Threads: NG * 8 consumer warps, then the producer warp, then the epilogue warp.
// PROBE: bandwidth probe - the bytes move through the ring exactly as usual, the consumers skip the arithmetic (the
// output is all zeros); it measures what the data path alone sustains for a shape.
template <int QT, typename T, int MXC, int NG, int D, bool PROBE>
__global__ void __launch_bounds__((NG * kGroupWarps + 2) * 32, NG == 1 ? 2 : 1)
gemv_stream_kernel(const T* __restrict__ x, const uint8_t* __restrict__ w, const T* __restrict__ bias, T* __restrict__ y,
                       int m, int n, int k, int* status, float* __restrict__ partial, int* __restrict__ flags, int mode, const PeerOut peers) {
  using MT = MmaType<T>;
  constexpr int NCW = NG * kGroupWarps;
  constexpr int MC = MXC == 1 ? 1 : 2;             // accumulator columns a lane keeps
  constexpr int kSbBytes = Geom<QT>::kSbBytes, kPitch = Geom<QT>::kPitch, kStageBytes = kRows * kPitch;
  constexpr bool kB32 = is_blk32<QT>();            // Q4_0 / MXFP4: one scale per 32 weights, two MMAs per block
  constexpr bool kNv = QT == QTYPE_NVFP4;          // a ue4m3 scale per 16 weights, multiplied into the operand (exact)
  constexpr bool kQ23 = is_q23<QT>();              // Q2_K / Q3_K: one MMA per 16-weight sub-block, offsets folded against 16-wide activation sums
  constexpr int kXG = kQ23 ? 16 : 32;              // activations per entry of the sum table sX
  constexpr bool kMinTerm = QT == QTYPE_Q4_K || QT == QTYPE_Q5_K || QT == QTYPE_Q4_0 || kQ23;   // these fold their mins / offsets against activation sums; Q6_K and the FP4 types have none
  constexpr bool kQ5 = QT == QTYPE_Q5_K;           // Q4_K arithmetic plus the fifth bit of every quant
  // From four activation rows on, the types with folded offsets take the per-sub-block activation sums from the tensor cores (an MMA of the same
  // activation fragment against an all-ones operand) instead of a table that every CTA builds from the whole activation
  // matrix before it starts: that prologue grows with M * K per CTA and cost a third of the launch at M = 8, K = 14336.
  constexpr bool kOnes = kMinTerm && MXC >= 4;
  constexpr bool kNeedK = kOnes && (QT == QTYPE_Q4_K || QT == QTYPE_Q5_K || QT == QTYPE_Q2_K);   // types with a min besides the operand offset
  constexpr int kQsOff = kQ5 ? 48 : 16;            // where the nibbles start inside a block
  static_assert(D % NG == 0 && D >= 2 * NG, "every group needs its own ring slots, at least two");
  static_assert(MXC == 1 || MXC == 2 || MXC == 4 || MXC == 8, "MXC");
  using Red = RedBuf<MXC, NCW>;

  extern __shared__ __align__(128) uint8_t smem_dyn[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_dyn);               // full[D], empty[D], red_full[2], red_empty[2]
  uint8_t* sW = smem_dyn + kBarBytes;                                         // D x kStageBytes
  Red* sRed = reinterpret_cast<Red*>(sW + size_t(D) * kStageBytes);      // [2]
  float* sX = reinterpret_cast<float*>(sRed + 2);                        // [MXC][k/32]
  __shared__ __align__(16) float sS[NCW][kRows][(QT == QTYPE_Q6_K || kQ23) ? kQ6ScalePitch : 8];   // d * sc per row, sub-block (warp-private scratch)
  __shared__ __align__(16) float sK[kNeedK ? NCW : 1][kNeedK ? kRows : 1][QT == QTYPE_Q2_K ? kQ6ScalePitch : 8];   // kOnes: MAGIC * d * sc + dmin * min (Q2_K: dmin * min) per row, sub-block
  __shared__ float sOut[kRows * MXC];                                    // epilogue warp scratch
  __shared__ int s_abort;
  static_assert((2 * D + 4) * 8 <= kBarBytes, "barrier area");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nsb = k >> 8, nsub = k / kXG;
  const int nchunks = (nsb + kKC - 1) / kKC;
  const int tiles = (n + kRows - 1) / kRows;
  // this CTA's units [u0, u1) of the tile-major line; walked from u1 - 1 down
  const int64_t total_units = int64_t(tiles) * nchunks;
  const bool descending = (mode & 1) != 0, unit_split = (mode & 2) != 0;
  const int u0 = unit_split ? int((int64_t(blockIdx.x) * total_units) / gridDim.x) : tile_begin(blockIdx.x, tiles, gridDim.x) * nchunks;
  const int u1 = unit_split ? int((int64_t(blockIdx.x + 1) * total_units) / gridDim.x) : tile_begin(blockIdx.x + 1, tiles, gridDim.x) * nchunks;
  const int nunits = u1 - u0;
  const int t_hi = (u1 - 1) / nchunks, t_lo = u0 / nchunks;
  const int ntiles = t_hi - t_lo + 1;               // tiles touched
  // a tile cut between two CTAs: the CTA that walks it FIRST leaves a partial, the one that walks it LAST adds it and stores
  const bool hi_cut = u1 % nchunks != 0, lo_cut = u0 % nchunks != 0;
  const bool first_cut = descending ? hi_cut : lo_cut, last_cut = descending ? lo_cut : hi_cut;
  const int other = descending ? int(blockIdx.x) - 1 : int(blockIdx.x) + 1;     // the CTA whose partial this one adds
  const int g_first = descending ? u1 - 1 : u0, dir = descending ? -1 : 1;
  const int64_t row_bytes = int64_t(nsb) * kSbBytes;
  volatile int* abort_flag = &s_abort;

  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * uint32_t(s); };
  auto empty = [&](int s) { return bar0 + 8u * uint32_t(D + s); };
  auto red_full = [&](int b) { return bar0 + 8u * uint32_t(2 * D + b); };
  auto red_empty = [&](int b) { return bar0 + 8u * uint32_t(2 * D + 2 + b); };

  if (tid == 0) {
    for (int s = 0; s < D; ++s) {
      mbar_init(full(s), 1);                    // the producer's arrive.expect_tx; the bytes complete the phase
      mbar_init(empty(s), kGroupWarps);         // one elected arrive per consumer warp of the slot's group
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(red_full(b), NCW);
      mbar_init(red_empty(b), 1);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

  if (warp == NCW) {
    // ------------------------------------------------------------------ producer: weights are constants, no dependency wait
    bool ok = true;
    int issued = 0, tile = g_first / nchunks, chunk = g_first % nchunks;
    const uint32_t sW_u32 = smem_u32(sW);
    for (int u = 0; u < nunits; ++u) {
      const int slot = u % D, it = u / D;
      if (it > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(empty(slot), uint32_t(it - 1) & 1u, abort_flag, status, ST_STREAM_EMPTY) ? 1 : 0) != 0;
        if (!ok) break;
      }
      const int sbs = min(kKC, nsb - chunk * kKC);
      const int rows_valid = min(kRows, n - tile * kRows);
      const uint32_t bytes_row = uint32_t(sbs) * kSbBytes;
      if (lane == 0) mbar_arrive_expect_tx(full(slot), uint32_t(rows_valid) * bytes_row);
      __syncwarp();
      if (lane < rows_valid)
        bulk_load(sW_u32 + uint32_t(slot) * kStageBytes + uint32_t(lane) * kPitch,
                  w + int64_t(tile * kRows + lane) * row_bytes + int64_t(chunk) * (kKC * kSbBytes), bytes_row, full(slot));
      issued = u + 1;
      chunk += dir;
      if (chunk < 0) { chunk = nchunks - 1; --tile; }
      else if (chunk == nchunks) { chunk = 0; ++tile; }
    }
    if (!ok && lane == 0)       // aborting: the copies still in flight must land before this CTA's shared memory goes away
      for (int v = max(0, issued - D); v < issued; ++v) mbar_wait_plain(full(v % D), uint32_t(v / D) & 1u);
    return;
  }

  // Everything below reads activations / writes outputs that a preceding kernel in the stream may still be producing.
  asm volatile("griddepcontrol.wait;\n" ::: "memory");

  if (warp == NCW + 1) {
    // ------------------------------------------------------------------ epilogue warp
    __shared__ float sPart[kRows * 8];      // the neighbouring CTA's partial sums of the cut tile, fetched as soon as they exist
    bool have_partial = !last_cut;
    // Fetches the neighbour's partial if its flag is up (blocking = keep polling, bounded); all lanes return the same answer.
    auto fetch_partial = [&](bool blocking) -> bool {
      const int* flag = flags + other;
      int seen = 0;
      if (lane == 0) {
        seen = ld_acquire_gpu(flag) != 0;
        if (!seen && blocking) {
          const uint64_t start = globaltimer_ns();
          for (uint32_t i = 0; i < kSpinLimit && !seen; ++i) {
            __nanosleep(40);
            seen = ld_acquire_gpu(flag) != 0;
            if (!seen && (i & 63u) == 63u && (*abort_flag || globaltimer_ns() - start > kWaitLimitNs)) break;
          }
          if (!seen) { *abort_flag = 1; atomicCAS(status, 0, ST_STREAM_PARTIAL); }
        }
      }
      seen = __shfl_sync(0xffffffffu, seen, 0);
      if (!seen) return false;
      const float* theirs = partial + size_t(other) * (kRows * 8);
      for (int idx = lane; idx < kRows * MXC; idx += 32) sPart[idx] = __ldcg(theirs + idx);
      __syncwarp();
      if (lane == 0) st_release_gpu(flags + other, 0);      // lowered by its only reader: nothing to clear between launches
      return true;
    };
    for (int tl = 0; tl < ntiles; ++tl) {
      const int buf = tl & 1;
      if (!have_partial) have_partial = fetch_partial(false);      // off the critical path: the neighbour wrote it at its start
      if (!(__all_sync(0xffffffffu, mbar_wait(red_full(buf), uint32_t(tl >> 1) & 1u, abort_flag, status, ST_STREAM_RED_FULL) ? 1 : 0))) break;
      const Red& rb = sRed[buf];
      for (int idx = lane; idx < kRows * MXC; idx += 32) {
        const int r = idx & (kRows - 1), c = idx >> 4;
        float v = 0.f, xs = 0.f;
#pragma unroll
        for (int wv = 0; wv < NCW; ++wv) {
          v += rb.red[wv][r][c];
          xs += rb.xt[wv][r][c];
        }
        sOut[idx] = v - xs;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(red_empty(buf));
      const int tile = descending ? t_hi - tl : t_lo + tl;
      if (tl == 0 && first_cut) {
        // the rest of this tile belongs to the neighbouring CTA, which reaches it last: leave the partial sums, raise the flag
        float* mine = partial + size_t(blockIdx.x) * (kRows * 8);
        for (int idx = lane; idx < kRows * MXC; idx += 32) mine[idx] = sOut[idx];
        __threadfence();
        __syncwarp();
        if (lane == 0) st_release_gpu(flags + blockIdx.x, 1);
        continue;
      }
      if (tl == ntiles - 1 && last_cut) {
        // the other chunks of this tile were computed by the neighbouring CTA at the start of its walk
        if (!have_partial) have_partial = fetch_partial(true);
        if (!have_partial) break;
        for (int idx = lane; idx < kRows * MXC; idx += 32) sOut[idx] += sPart[idx];
        __syncwarp();
      }
      for (int idx = lane; idx < kRows * MXC; idx += 32) {
        const int r = idx & (kRows - 1), c = idx >> 4;
        const int row = tile * kRows + r;
        if (row >= n || c >= m) continue;
        float v = sOut[idx];
        int64_t at = int64_t(c) * n + row;
        if (peers.act != ACT_NONE) {
          // gated pair: rows r < 8 of the tile belong to the first matrix, r + 8 to the second; output has n / 2 columns
          if (r >= 8) continue;
          float u = sOut[idx + 8];
          if (bias != nullptr) {           // interleaved like the rows: bias0 of the gate row, bias1 of its up row
            v += MT::to_float(bias[row]);
            u += MT::to_float(bias[row + 8]);
          }
          v = gate_activation(v, peers.act) * u;
          at = int64_t(c) * (n >> 1) + (tile * 8 + r);
        } else if (bias != nullptr) {
          v += MT::to_float(bias[row]);
        }
        const T out = MT::from_float(v);
        y[at] = out;
#pragma unroll
        for (int pi = 0; pi < 8; ++pi)
          if (pi < peers.count) static_cast<T*>(peers.ptr[pi])[at] = out;
      }
      __syncwarp();                         // sOut is rewritten for the next tile
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  const int cw = warp, grp = cw / kGroupWarps, wq = cw % kGroupWarps;
  const int g = lane >> 2, t = lane & 3;
  const int srow = lane >> 1, shalf = lane & 1;   // scale-decode role of this lane

  // X[c][j] = sum of activations of row c over sub-block j (rows >= m are zero)
  for (int i = tid; kMinTerm && !kOnes && i < nsub * MXC; i += NCW * 32) {
    const int c = i / nsub, j = i - c * nsub;
    float s = 0.f;
    if (c < m) {
      const uint4* px = reinterpret_cast<const uint4*>(x + int64_t(c) * k + int64_t(j) * kXG);
#pragma unroll
      for (int q = 0; q < kXG / 8; ++q) s += MT::sum8(__ldg(px + q));
    }
    sX[i] = s;
  }
  named_barrier(1, NCW * 32);

  float res[1][4] = {{0.f, 0.f, 0.f, 0.f}};
  float zero4[4];
  opaque_zero4(zero4);
  float xt[MXC];
#pragma unroll
  for (int c = 0; c < MXC; ++c) xt[c] = 0.f;
  const T* xbase = x + int64_t(min(g, m - 1)) * k;   // rows >= m read a clamped (valid) row; their columns are never stored
  const T* xrow = xbase + 8 * t;

  bool ok = true;
  int cur_tile = 0;                             // tile (local index) the accumulators belong to
  auto flush = [&](int tl) {
    const int buf = tl & 1;
    if (tl >= 2) ok = __all_sync(0xffffffffu, mbar_wait(red_empty(buf), uint32_t((tl >> 1) - 1) & 1u, abort_flag, status, ST_STREAM_RED_EMPTY) ? 1 : 0) != 0;
    if (!ok) return;
    Red& rb = sRed[buf];
    if (2 * t < MXC) {
      rb.red[cw][g][2 * t] = res[0][0];
      rb.red[cw][g + 8][2 * t] = res[0][2];
      if (MC == 2) {
        rb.red[cw][g][2 * t + 1] = res[0][1];
        rb.red[cw][g + 8][2 * t + 1] = res[0][3];
      }
    }
#pragma unroll
    for (int c = 0; c < MXC; ++c) {
      const float both = (kMinTerm && !kOnes) ? xt[c] + __shfl_xor_sync(0xffffffffu, xt[c], 1) : 0.f;
      if (shalf == 0) rb.xt[cw][srow][c] = both;
      xt[c] = 0.f;
    }
    res[0][0] = res[0][1] = res[0][2] = res[0][3] = 0.f;
    __syncwarp();
    if (lane == 0) mbar_arrive(red_full(buf));
  };

  // local unit u is global unit g_first + dir * u: its chunk moves by dir, its local tile index counts up
  int tl = 0, chunk = g_first % nchunks + dir * grp;
  while (chunk < 0 && tl < ntiles) { chunk += nchunks; ++tl; }
  while (chunk >= nchunks && tl < ntiles) { chunk -= nchunks; ++tl; }
  for (int u = grp; u < nunits && ok; u += NG) {
    while (cur_tile < tl && ok) { flush(cur_tile); ++cur_tile; }
    if (!ok) break;
    const int slot = u % D;
    ok = __all_sync(0xffffffffu, mbar_wait(full(slot), uint32_t(u / D) & 1u, abort_flag, status, ST_STREAM_FULL) ? 1 : 0) != 0;
    if (!ok) break;
    const int sb = chunk * kKC + wq;
    if (!PROBE && sb < nsb && kB32) {
      if constexpr (kB32) {
        constexpr int BB = QT == QTYPE_Q4_0 ? 18 : 17, QOFF = BB - 16;       // block bytes, where its 16 nibble bytes start
        const uint8_t* st = sW + size_t(slot) * kStageBytes + wq * kSbBytes;
        {  // lane pair (srow, shalf): the scales of blocks 4*shalf .. +3 of row srow -> shared memory; Q4_0's offset folded against X
          const uint8_t* sp = st + srow * kPitch + 4 * shalf * BB;
          float4 dsv;
          float* dsf = reinterpret_cast<float*>(&dsv);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if constexpr (QT == QTYPE_Q4_0) dsf[i] = half_bits_to_float(*reinterpret_cast<const uint16_t*>(sp + BB * i));
            else dsf[i] = __fmul_rn(e8m0_half(sp[BB * i]), 2.f);             // 2^(e - 127): the operands are the e2m1 values themselves
          }
          *reinterpret_cast<float4*>(&sS[cw][srow][4 * shalf]) = dsv;
          if constexpr (kMinTerm && !kOnes) {
            constexpr float kOff = MT::kMagic + 8.f;                          // operand = MAGIC + q, weight = d * (q - 8)
#pragma unroll
            for (int c = 0; c < MXC; ++c) {
              const float4 X = *reinterpret_cast<const float4*>(&sX[c * nsub + sb * 8 + 4 * shalf]);
              xt[c] = fmaf(kOff * dsf[0], X.x, xt[c]);
              xt[c] = fmaf(kOff * dsf[1], X.y, xt[c]);
              xt[c] = fmaf(kOff * dsf[2], X.z, xt[c]);
              xt[c] = fmaf(kOff * dsf[3], X.w, xt[c]);
            }
          }
        }
        __syncwarp();
        const float4 dsa0 = *reinterpret_cast<const float4*>(&sS[cw][g][0]);
        const float4 dsa1 = *reinterpret_cast<const float4*>(&sS[cw][g][4]);
        const float4 dsb0 = *reinterpret_cast<const float4*>(&sS[cw][g + 8][0]);
        const float4 dsb1 = *reinterpret_cast<const float4*>(&sS[cw][g + 8][4]);
        const float ds_a[8] = {dsa0.x, dsa0.y, dsa0.z, dsa0.w, dsa1.x, dsa1.y, dsa1.z, dsa1.w};
        const float ds_b[8] = {dsb0.x, dsb0.y, dsb0.z, dsb0.w, dsb1.x, dsb1.y, dsb1.z, dsb1.w};
        // Byte j of a block holds weight j (low nibble) and weight 16 + j (high nibble).  Lane t takes bytes 4t .. 4t+3 of rows g
        // and g + 8: its low nibbles are weights 4t .. 4t+3 (first MMA of the block: K slots 2t, 2t+1 and 2t+8, 2t+9), its high
        // nibbles weights 16 + 4t .. (second MMA); the activations follow the same order (two 8-byte loads per block).
        const uint8_t* r0 = st + g * kPitch + 4 * t;
        const uint8_t* r1 = r0 + 8 * kPitch;
        const T* xs = xbase + 4 * t + sb * 256;
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          const int o = BB * b + QOFF, oa = o & ~3, sh = 8 * (o & 3);         // constants after unrolling; blocks are 1- / 2-byte aligned
          uint32_t w0 = *reinterpret_cast<const uint32_t*>(r0 + oa), w1 = *reinterpret_cast<const uint32_t*>(r1 + oa);
          if (sh != 0) {
            w0 = __funnelshift_r(w0, *reinterpret_cast<const uint32_t*>(r0 + oa + 4), sh);
            w1 = __funnelshift_r(w1, *reinterpret_cast<const uint32_t*>(r1 + oa + 4), sh);
          }
          uint32_t a_lo[4], a_hi[4];
          if constexpr (QT == QTYPE_Q4_0) {
            const uint32_t l0 = w0 & 0x0f0f0f0fu, h0 = (w0 >> 4) & 0x0f0f0f0fu, l1 = w1 & 0x0f0f0f0fu, h1 = (w1 >> 4) & 0x0f0f0f0fu;
            a_lo[0] = MT::fix(__byte_perm(l0, MT::kMagicBytes, 0x4140)); a_lo[1] = MT::fix(__byte_perm(l1, MT::kMagicBytes, 0x4140));
            a_lo[2] = MT::fix(__byte_perm(l0, MT::kMagicBytes, 0x4342)); a_lo[3] = MT::fix(__byte_perm(l1, MT::kMagicBytes, 0x4342));
            a_hi[0] = MT::fix(__byte_perm(h0, MT::kMagicBytes, 0x4140)); a_hi[1] = MT::fix(__byte_perm(h1, MT::kMagicBytes, 0x4140));
            a_hi[2] = MT::fix(__byte_perm(h0, MT::kMagicBytes, 0x4342)); a_hi[3] = MT::fix(__byte_perm(h1, MT::kMagicBytes, 0x4342));
          } else {
            fp4x8_operands<T>(w0, a_lo[0], a_lo[2], a_hi[0], a_hi[2]);
            fp4x8_operands<T>(w1, a_lo[1], a_lo[3], a_hi[1], a_hi[3]);
          }
          const uint2 xa = __ldg(reinterpret_cast<const uint2*>(xs + 32 * b));
          const uint2 xb = __ldg(reinterpret_cast<const uint2*>(xs + 32 * b + 16));
          float acc[4];
          MT::mma_c(acc, a_lo, xa.x, xa.y, zero4);
          MT::mma(acc, a_hi, xb.x, xb.y);
          if constexpr (kOnes) {               // Q4_0: sum of (MAGIC + q) x  ->  sum of (q - 8) x with the block's activation sums
            const uint32_t ones[4] = {MT::kOnePair, MT::kOnePair, MT::kOnePair, MT::kOnePair};
            float sx[4];
            MT::mma_c(sx, ones, xa.x, xa.y, zero4);
            MT::mma(sx, ones, xb.x, xb.y);
            constexpr float kOff = MT::kMagic + 8.f;
            acc[0] = fmaf(-kOff, sx[0], acc[0]);
            acc[2] = fmaf(-kOff, sx[0], acc[2]);
            if (MC == 2) {
              acc[1] = fmaf(-kOff, sx[1], acc[1]);
              acc[3] = fmaf(-kOff, sx[1], acc[3]);
            }
          }
          res[0][0] = fmaf(ds_a[b], acc[0], res[0][0]);
          res[0][2] = fmaf(ds_b[b], acc[2], res[0][2]);
          if (MC == 2) {
            res[0][1] = fmaf(ds_a[b], acc[1], res[0][1]);
            res[0][3] = fmaf(ds_b[b], acc[3], res[0][3]);
          }
        }
      }
    } else if (!PROBE && sb < nsb && kQ23) {
      if constexpr (kQ23) {
        // Q2_K: scales[16] (4-bit scale, 4-bit min per 16 weights), qs[64], d, dmin.  Q3_K: hmask[32], qs[64], scales[12] (6-bit), d.
        // Weight 128*hb + 32*j + l is bits 2j, 2j+1 of qs[32*hb + l] (Q3_K: plus bit 4*hb + j of hmask[l] as a third bit, less 4);
        // sub-block (hb, j, h16) = its weights l = 16*h16 .. +15, scale index 8*hb + 2*j + h16.  One MMA per sub-block.
        constexpr int kQs = QT == QTYPE_Q2_K ? 16 : 32;
        const uint8_t* st = sW + size_t(slot) * kStageBytes + wq * kSbBytes;
        {  // lane pair (srow, shalf): the eight sub-block scales of half-block shalf of row srow
          const uint8_t* blk = st + srow * kPitch;
          float dsf[8], kk[8], dmv[8];         // d * scale; folded offset + min; Q2_K: dmin * min alone
          if constexpr (QT == QTYPE_Q2_K) {
            const float d = half_at(blk + 80), dmin = half_at(blk + 82);
            const uint32_t* scp = reinterpret_cast<const uint32_t*>(blk + 8 * shalf);   // blocks (84 B) are word aligned, not more
            const uint32_t sc0 = scp[0], sc1 = scp[1];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t b = ((i < 4 ? sc0 : sc1) >> (8 * (i & 3))) & 0xffu;
              dsf[i] = d * float(b & 0x0fu);
              dmv[i] = dmin * float(b >> 4);
              kk[i] = fmaf(MT::kMagic, dsf[i], dmv[i]);
            }
          } else {
            const float d = half_at(blk + 108);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              dsf[i] = d * float(q3k_scale(blk + 96, 8 * shalf + i) - 32);
              dmv[i] = 0.f;
              kk[i] = (MT::kMagic + 4.f) * dsf[i];                                    // operand = MAGIC + (q + 4)
            }
          }
          *reinterpret_cast<float4*>(&sS[cw][srow][8 * shalf]) = make_float4(dsf[0], dsf[1], dsf[2], dsf[3]);
          *reinterpret_cast<float4*>(&sS[cw][srow][8 * shalf + 4]) = make_float4(dsf[4], dsf[5], dsf[6], dsf[7]);
          if constexpr (kNeedK) {                 // Q2_K: dmin * min, applied to the sums from the tensor cores below
            *reinterpret_cast<float4*>(&sK[cw][srow][8 * shalf]) = make_float4(dmv[0], dmv[1], dmv[2], dmv[3]);
            *reinterpret_cast<float4*>(&sK[cw][srow][8 * shalf + 4]) = make_float4(dmv[4], dmv[5], dmv[6], dmv[7]);
          }
#pragma unroll
          for (int c = 0; c < (kOnes ? 0 : MXC); ++c) {
            const float4 X0 = *reinterpret_cast<const float4*>(&sX[c * nsub + sb * 16 + 8 * shalf]);
            const float4 X1 = *reinterpret_cast<const float4*>(&sX[c * nsub + sb * 16 + 8 * shalf + 4]);
            const float X[8] = {X0.x, X0.y, X0.z, X0.w, X1.x, X1.y, X1.z, X1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) xt[c] = fmaf(kk[i], X[i], xt[c]);
          }
        }
        __syncwarp();
        // Lane t takes bytes 4t .. 4t+3 of every 16-byte run of rows g and g + 8: four weights of each of the four sub-blocks
        // (j = 0..3) that share those bytes; K slots 2t, 2t+1 and 2t+8, 2t+9 carry them, the activations follow the same order.
        // Q3_K blocks (110 B) sit 2 bytes off a word boundary in every odd super-block: two aligned loads and a funnel shift.
        const uint32_t sh = (QT == QTYPE_Q3_K) ? 16u * uint32_t(wq & 1) : 0u;
        auto word = [&](const uint8_t* p) -> uint32_t {      // 4 bytes at p, p being `sh / 8` bytes past a word boundary
          if constexpr (QT == QTYPE_Q3_K) {
            const uint32_t* a = reinterpret_cast<const uint32_t*>(p - (sh >> 3));
            return __funnelshift_r(a[0], a[1], sh);
          } else {
            return *reinterpret_cast<const uint32_t*>(p);
          }
        };
        const uint8_t* r0 = st + g * kPitch + 4 * t;
        const uint8_t* r1 = r0 + 8 * kPitch;
        const T* xs = xbase + 4 * t + sb * 256;
#pragma unroll
        for (int h16 = 0; h16 < 2; ++h16) {
          uint32_t hm0 = 0, hm1 = 0;
          if constexpr (QT == QTYPE_Q3_K) { hm0 = word(r0 + 16 * h16); hm1 = word(r1 + 16 * h16); }
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            const uint32_t w0 = word(r0 + kQs + 32 * hb + 16 * h16), w1 = word(r1 + kQs + 32 * hb + 16 * h16);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t n0 = (w0 >> (2 * j)) & 0x03030303u, n1 = (w1 >> (2 * j)) & 0x03030303u;
              if constexpr (QT == QTYPE_Q3_K) {
                n0 |= ((hm0 >> (4 * hb + j)) & 0x01010101u) << 2;
                n1 |= ((hm1 >> (4 * hb + j)) & 0x01010101u) << 2;
              }
              const uint32_t a[4] = {MT::fix(__byte_perm(n0, MT::kMagicBytes, 0x4140)), MT::fix(__byte_perm(n1, MT::kMagicBytes, 0x4140)),
                                     MT::fix(__byte_perm(n0, MT::kMagicBytes, 0x4342)), MT::fix(__byte_perm(n1, MT::kMagicBytes, 0x4342))};
              const uint2 xa = __ldg(reinterpret_cast<const uint2*>(xs + 128 * hb + 32 * j + 16 * h16));
              float acc[4];
              MT::mma_c(acc, a, xa.x, xa.y, zero4);
              const int idx = 8 * hb + 2 * j + h16;
              const float da = sS[cw][g][idx], db = sS[cw][g + 8][idx];      // 16 scales per row: read where used, not held in registers
              if constexpr (kOnes) {             // the operand offset (and Q2_K's min) against the sub-block's activation sums
                const uint32_t ones[4] = {MT::kOnePair, MT::kOnePair, MT::kOnePair, MT::kOnePair};
                float sx[4];
                MT::mma_c(sx, ones, xa.x, xa.y, zero4);
                constexpr float kOff = MT::kMagic + (QT == QTYPE_Q3_K ? 4.f : 0.f);
                acc[0] = fmaf(-kOff, sx[0], acc[0]);
                acc[2] = fmaf(-kOff, sx[0], acc[2]);
                if (MC == 2) {
                  acc[1] = fmaf(-kOff, sx[1], acc[1]);
                  acc[3] = fmaf(-kOff, sx[1], acc[3]);
                }
                if constexpr (QT == QTYPE_Q2_K) {
                  const float ma = sK[cw][g][idx], mb = sK[cw][g + 8][idx];
                  res[0][0] = fmaf(-ma, sx[0], res[0][0]);
                  res[0][2] = fmaf(-mb, sx[0], res[0][2]);
                  if (MC == 2) {
                    res[0][1] = fmaf(-ma, sx[1], res[0][1]);
                    res[0][3] = fmaf(-mb, sx[1], res[0][3]);
                  }
                }
              }
              res[0][0] = fmaf(da, acc[0], res[0][0]);
              res[0][2] = fmaf(db, acc[2], res[0][2]);
              if (MC == 2) {
                res[0][1] = fmaf(da, acc[1], res[0][1]);
                res[0][3] = fmaf(db, acc[3], res[0][3]);
              }
            }
          }
        }
      }
    } else if (!PROBE && sb < nsb && kNv) {
      if constexpr (kNv) {
        // Four blocks of 64 weights (four ue4m3 scales, 32 bytes of nibbles).  Lane t owns sub-block t of every block for rows g
        // and g + 8: 8 bytes whose byte i holds weights i (low nibble) and 8 + i (high nibble).  Value x scale is exact in either
        // 16-bit type (2 + 4 significant bits), so the operand is the dequantized weight itself and nothing is applied after
        // the MMA; the four MMAs of a block take weights 4j .. 4j+3 of every sub-block (K slots 2t, 2t+1, 2t+8, 2t+9), the
        // activations follow the same order: 16 consecutive values per lane and block.
        const uint8_t* st = sW + size_t(slot) * kStageBytes + wq * kSbBytes;
        const uint8_t* r0 = st + g * kPitch;
        const uint8_t* r1 = r0 + 8 * kPitch;
        const T* xs = xbase + sb * 256 + 16 * t;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const uint32_t s0 = splat_pair<T>(__fmul_rn(ue4m3_half(r0[36 * b + t]), 2.f));
          const uint32_t s1 = splat_pair<T>(__fmul_rn(ue4m3_half(r1[36 * b + t]), 2.f));
          uint32_t a[4][4];           // [MMA j][fragment register]
#pragma unroll
          for (int i = 0; i < 2; ++i) {   // word i: low nibbles -> MMA i, high nibbles -> MMA 2 + i
            const uint32_t w0 = *reinterpret_cast<const uint32_t*>(r0 + 36 * b + 4 + 8 * t + 4 * i);
            const uint32_t w1 = *reinterpret_cast<const uint32_t*>(r1 + 36 * b + 4 + 8 * t + 4 * i);
            fp4x8_operands<T>(w0, a[i][0], a[i][2], a[2 + i][0], a[2 + i][2]);
            fp4x8_operands<T>(w1, a[i][1], a[i][3], a[2 + i][1], a[2 + i][3]);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            a[j][0] = mul_pair<T>(a[j][0], s0); a[j][2] = mul_pair<T>(a[j][2], s0);
            a[j][1] = mul_pair<T>(a[j][1], s1); a[j][3] = mul_pair<T>(a[j][3], s1);
          }
          const uint4 xa = __ldg(reinterpret_cast<const uint4*>(xs + 64 * b));
          const uint4 xb = __ldg(reinterpret_cast<const uint4*>(xs + 64 * b + 8));
          float acc[4];
          MT::mma_c(acc, a[0], xa.x, xa.y, zero4);
          MT::mma(acc, a[1], xa.z, xa.w);
          MT::mma(acc, a[2], xb.x, xb.y);
          MT::mma(acc, a[3], xb.z, xb.w);
          res[0][0] += acc[0];
          res[0][2] += acc[2];
          if (MC == 2) {
            res[0][1] += acc[1];
            res[0][3] += acc[3];
          }
        }
      }
    } else if (!PROBE && sb < nsb && QT == QTYPE_Q6_K) {
      if constexpr (QT == QTYPE_Q6_K) {
        // row pitch and stage size are multiples of 4, so a block's phase against a word boundary is that of wq * 210
        const uint8_t* st = sW + size_t(slot) * kStageBytes + wq * kSbBytes;
        const T* const xr[1] = {xbase + 4 * t};                // this lane's four K positions of every 16-wide sub-block
        if (wq & 1)
          q6k_superblock<T, 1, MC, Q6_ODD>(st + srow * kPitch, st + g * kPitch, st + (g + 8) * kPitch, sS[cw], xr, sb, lane, res);
        else
          q6k_superblock<T, 1, MC, Q6_ALIGNED>(st + srow * kPitch, st + g * kPitch, st + (g + 8) * kPitch, sS[cw], xr, sb, lane, res);
      }
    } else if (!PROBE && sb < nsb && !kB32 && !kNv && !kQ23) {
      const uint8_t* st = sW + size_t(slot) * kStageBytes + wq * kSbBytes;
      {  // lane pair (srow, shalf): 4 sub-block scales -> ds to shared memory, min/MAGIC term folded against X
        const uint4 hdr = *reinterpret_cast<const uint4*>(st + srow * kPitch);
        const float d = half_bits_to_float(uint16_t(hdr.x & 0xffffu));
        const float dmin = half_bits_to_float(uint16_t(hdr.x >> 16));
        // sub-blocks 0..3 keep their 6-bit fields in place; 4..7 are split across two bytes
        const uint32_t sc_lo = hdr.y & 0x3f3f3f3fu, mn_lo = hdr.z & 0x3f3f3f3fu;
        const uint32_t sc_hi = (hdr.w & 0x0f0f0f0fu) | (((hdr.y >> 6) & 0x03030303u) << 4);
        const uint32_t mn_hi = ((hdr.w >> 4) & 0x0f0f0f0fu) | (((hdr.z >> 6) & 0x03030303u) << 4);
        const uint32_t scb = shalf ? sc_hi : sc_lo, mnb = shalf ? mn_hi : mn_lo;
        float4 dsv;
        float kk[4];
        float* dsf = reinterpret_cast<float*>(&dsv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          dsf[i] = d * byte_to_float(scb, i);
          kk[i] = fmaf(MT::kMagic, dsf[i], dmin * byte_to_float(mnb, i));
        }
        *reinterpret_cast<float4*>(&sS[cw][srow][4 * shalf]) = dsv;
        if constexpr (kOnes) {
          *reinterpret_cast<float4*>(&sK[cw][srow][4 * shalf]) = make_float4(kk[0], kk[1], kk[2], kk[3]);
        } else {
#pragma unroll
          for (int c = 0; c < MXC; ++c) {
            const float4 X = *reinterpret_cast<const float4*>(&sX[c * nsub + sb * 8 + 4 * shalf]);
            xt[c] = fmaf(kk[0], X.x, xt[c]);
            xt[c] = fmaf(kk[1], X.y, xt[c]);
            xt[c] = fmaf(kk[2], X.z, xt[c]);
            xt[c] = fmaf(kk[3], X.w, xt[c]);
          }
        }
      }
      __syncwarp();
      const float4 dsa0 = *reinterpret_cast<const float4*>(&sS[cw][g][0]);
      const float4 dsa1 = *reinterpret_cast<const float4*>(&sS[cw][g][4]);
      const float4 dsb0 = *reinterpret_cast<const float4*>(&sS[cw][g + 8][0]);
      const float4 dsb1 = *reinterpret_cast<const float4*>(&sS[cw][g + 8][4]);
      const float ds_a[8] = {dsa0.x, dsa0.y, dsa0.z, dsa0.w, dsa1.x, dsa1.y, dsa1.z, dsa1.w};
      const float ds_b[8] = {dsb0.x, dsb0.y, dsb0.z, dsb0.w, dsb1.x, dsb1.y, dsb1.z, dsb1.w};
      const uint8_t* q0p = st + g * kPitch + kQsOff + 8 * t;
      const uint8_t* q1p = q0p + 8 * kPitch;
      const T* xs = xrow + sb * 256;
      // Q5_K: bit 2G+h of qh byte l is the fifth bit of weight l of sub-block 2G+h; this lane's eight l are bytes 8t .. 8t+7
      uint2 qh0 = make_uint2(0u, 0u), qh1 = make_uint2(0u, 0u);
      if constexpr (kQ5) {
        qh0 = *reinterpret_cast<const uint2*>(st + g * kPitch + 16 + 8 * t);
        qh1 = *reinterpret_cast<const uint2*>(st + (g + 8) * kPitch + 16 + 8 * t);
      }
#pragma unroll
      for (int G = 0; G < 4; ++G) {
        const uint2 q0 = *reinterpret_cast<const uint2*>(q0p + 32 * G);
        const uint2 q1 = *reinterpret_cast<const uint2*>(q1p + 32 * G);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t n0x = (h ? q0.x >> 4 : q0.x) & 0x0f0f0f0fu, n0y = (h ? q0.y >> 4 : q0.y) & 0x0f0f0f0fu;
          uint32_t n1x = (h ? q1.x >> 4 : q1.x) & 0x0f0f0f0fu, n1y = (h ? q1.y >> 4 : q1.y) & 0x0f0f0f0fu;
          if constexpr (kQ5) {               // q = nibble + 16 * bit: still an exact 128 + q operand (q <= 31)
            constexpr uint32_t kBit = 0x01010101u;
            n0x |= ((qh0.x >> (2 * G + h)) & kBit) * 16u;
            n0y |= ((qh0.y >> (2 * G + h)) & kBit) * 16u;
            n1x |= ((qh1.x >> (2 * G + h)) & kBit) * 16u;
            n1y |= ((qh1.y >> (2 * G + h)) & kBit) * 16u;
          }
          const uint32_t a_lo[4] = {MT::fix(__byte_perm(n0x, MT::kMagicBytes, 0x4140)), MT::fix(__byte_perm(n1x, MT::kMagicBytes, 0x4140)),
                                    MT::fix(__byte_perm(n0x, MT::kMagicBytes, 0x4342)), MT::fix(__byte_perm(n1x, MT::kMagicBytes, 0x4342))};
          const uint32_t a_hi[4] = {MT::fix(__byte_perm(n0y, MT::kMagicBytes, 0x4140)), MT::fix(__byte_perm(n1y, MT::kMagicBytes, 0x4140)),
                                    MT::fix(__byte_perm(n0y, MT::kMagicBytes, 0x4342)), MT::fix(__byte_perm(n1y, MT::kMagicBytes, 0x4342))};
          // rows >= m read a clamped (valid) row; their accumulator columns are never stored
          const uint4 xb = __ldg(reinterpret_cast<const uint4*>(xs + 64 * G + 32 * h));
          float acc[4];
          MT::mma_c(acc, a_lo, xb.x, xb.y, zero4);
          MT::mma(acc, a_hi, xb.z, xb.w);
          const float dsr0 = ds_a[2 * G + h], dsr1 = ds_b[2 * G + h];
          res[0][0] = fmaf(dsr0, acc[0], res[0][0]);
          res[0][2] = fmaf(dsr1, acc[2], res[0][2]);
          if (MC == 2) {
            res[0][1] = fmaf(dsr0, acc[1], res[0][1]);
            res[0][3] = fmaf(dsr1, acc[3], res[0][3]);
          }
          if constexpr (kOnes) {
            // the sub-block's activation sums of columns 2t, 2t+1 (the same in every row of the tile), then the folded offsets
            const uint32_t ones[4] = {MT::kOnePair, MT::kOnePair, MT::kOnePair, MT::kOnePair};
            float sx[4];
            MT::mma_c(sx, ones, xb.x, xb.y, zero4);
            MT::mma(sx, ones, xb.z, xb.w);
            const float kk0 = sK[cw][g][2 * G + h], kk1 = sK[cw][g + 8][2 * G + h];
            res[0][0] = fmaf(-kk0, sx[0], res[0][0]);
            res[0][2] = fmaf(-kk1, sx[0], res[0][2]);
            if (MC == 2) {
              res[0][1] = fmaf(-kk0, sx[1], res[0][1]);
              res[0][3] = fmaf(-kk1, sx[1], res[0][3]);
            }
          }
        }
      }
    }
    __syncwarp();                              // every lane is done with the stage (and with sS)
    if (lane == 0) mbar_arrive(empty(slot));
    chunk += dir * NG;
    while (chunk < 0) { chunk += nchunks; ++tl; }
    while (chunk >= nchunks) { chunk -= nchunks; ++tl; }
  }
  // the tiles this warp has not flushed yet (all of them contribute to every tile's reduction, zeros included)
  while (cur_tile < ntiles && ok) { flush(cur_tile); ++cur_tile; }
}

// ---------------------------------------------------------------------------------------- host side
int* stream_status_ptr() {
  static int* ptr[kGemvMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kGemvMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_stream_status) != cudaSuccess) return nullptr;
    ptr[dev] = static_cast<int*>(p);
  }
  return ptr[dev];
}

// Partial-tile workspace and flags: one set per (device, stream) - launches on one stream are ordered (a launch writes its
// partials only after the preceding kernel has completed, see griddepcontrol.wait above) and may share it, launches on
// different streams may overlap and must not.  kMaxCtas partial tiles of 16 x 8 floats and as many flag words, zeroed
// once; every flag a launch raises is lowered again by the CTA that consumes it.
constexpr int kMaxCtas = 1024;
struct Scratch { float* partial = nullptr; int* flags = nullptr; };
struct ScratchKey {
  int dev;
  cudaStream_t stream;
  bool operator<(const ScratchKey& o) const { return dev != o.dev ? dev < o.dev : stream < o.stream; }
};
static std::mutex g_scratch_mutex;
static std::map<ScratchKey, Scratch> g_scratch;

static int stream_scratch(cudaStream_t stream, Scratch* out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return RC_LAUNCH;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  Scratch& sc = g_scratch[ScratchKey{dev, stream}];
  if (sc.partial == nullptr) {
    // allocated outside of stream capture only: callers warm a shape up once before capturing a graph
    if (cudaMalloc(&sc.partial, size_t(kMaxCtas) * kRows * 8 * sizeof(float)) != cudaSuccess) return RC_LAUNCH;
    if (cudaMalloc(&sc.flags, size_t(kMaxCtas) * sizeof(int)) != cudaSuccess) { cudaFree(sc.partial); sc.partial = nullptr; return RC_LAUNCH; }
    cudaMemset(sc.flags, 0, size_t(kMaxCtas) * sizeof(int));
  }
  *out = sc;
  return RC_OK;
}

template <int QT, typename T, int MXC, int NG, int D, bool PROBE = false>
static int launch_cfg(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, int ctas_per_sm, const PeerOut& peers,
                          cudaStream_t s, int mode = 3) {     // mode: bit 0 = walk downwards, bit 1 = split at unit granularity
  const size_t smem = smem_fixed_bytes<QT, MXC, NG, D>() + (MXC >= 4 ? 0 : (QT == QTYPE_Q4_K || QT == QTYPE_Q5_K || QT == QTYPE_Q4_0) ? size_t(k / 32) * MXC * sizeof(float)
                      : is_q23<QT>() ? size_t(k / 16) * MXC * sizeof(float) : 0);      // the activation-sum table of the types that keep one
  if (smem > 216 * 1024) return RC_RANGE;            // + up to 9 KB of static shared memory, under the 227 KB per CTA
  int* status = stream_status_ptr();
  if (status == nullptr) return RC_LAUNCH;
  auto kern = gemv_stream_kernel<QT, T, MXC, NG, D, PROBE>;
  static SmemOptIn granted;
  if (!smem_opt_in(kern, smem, granted)) return RC_LAUNCH;
  int sm_count = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = (n + kRows - 1) / kRows;
  // never more CTAs than tiles: a CTA then owns at least one tile's worth of units, so a tile is cut between two CTAs at most
  const int ctas = min(min(tiles, sm_count * (ctas_per_sm < 1 ? 1 : ctas_per_sm)), kMaxCtas);
  Scratch sc;
  if (int rc = stream_scratch(s, &sc)) return rc;
  const cudaError_t err = gemv_launch(kern, ctas, 1, (NG * kGroupWarps + 2) * 32, smem, s, static_cast<const T*>(a),
                                      static_cast<const uint8_t*>(b), static_cast<const T*>(bias), static_cast<T*>(c), m, n, k, status,
                                      sc.partial, sc.flags, mode, peers);
  return err == cudaSuccess ? RC_OK : RC_LAUNCH;
}

// Tuning configurations (the `config` byte of a variant code, see dinoml_b200_gguf.h).  0 = the default for the shape.
//   1: 8 consumer warps, 5 ring slots (Q6_K: 4), one CTA per SM - two launches fit side by side on an SM
//   2: 16 consumer warps, 6 ring slots (Q6_K: 4), one CTA per SM
//   3: 16 consumer warps, 8 ring slots (Q6_K: 6), one CTA per SM
//   4: 8 consumer warps, 4 ring slots (Q6_K: 3), two CTAs per SM
// A Q6_K stage is 26.3 KB against 18.5 KB for Q4_K, hence the shallower rings.
// Bit 7 of the configuration byte (0x80 | 1..4) selects the bandwidth probe of that configuration (bfloat16, M = 1).
constexpr int kStreamConfigs = 4;
constexpr int kProbeBit = 0x80;
template <int QT, typename T, int MXC>
static int launch_m(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, int config, const PeerOut& peers,
                    cudaStream_t s) {
  constexpr bool Q6 = QT == QTYPE_Q6_K || QT == QTYPE_Q5_K;      // the larger stages (26.3 / 23.0 KB): shallower rings
  if (config & kProbeBit) {
    if constexpr (MXC == 1 && std::is_same<T, __nv_bfloat16>::value) {
      switch (config & ~kProbeBit) {
        case 1: return launch_cfg<QT, T, 1, 1, Q6 ? 4 : 5, true>(a, b, bias, c, m, n, k, 1, peers, s);
        case 2: return launch_cfg<QT, T, 1, 2, Q6 ? 4 : 6, true>(a, b, bias, c, m, n, k, 1, peers, s);
        case 3: return launch_cfg<QT, T, 1, 2, Q6 ? 6 : 8, true>(a, b, bias, c, m, n, k, 1, peers, s);
        case 4: return launch_cfg<QT, T, 1, 1, Q6 ? 3 : 4, true>(a, b, bias, c, m, n, k, 2, peers, s);
        default: return RC_RANGE;
      }
    }
    return RC_RANGE;
  }
  if (config == 0) {
    // default: two CTAs of 8 consumer warps per SM; a weight with fewer tiles than SMs runs one CTA of 16 consumer warps each
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    config = (n + kRows - 1) / kRows <= sms ? 2 : 4;
  }
  switch (config) {
    case 1: return launch_cfg<QT, T, MXC, 1, Q6 ? 4 : 5>(a, b, bias, c, m, n, k, 1, peers, s);
    case 2: return launch_cfg<QT, T, MXC, 2, Q6 ? 4 : 6>(a, b, bias, c, m, n, k, 1, peers, s);
    case 3: return launch_cfg<QT, T, MXC, 2, Q6 ? 6 : 8>(a, b, bias, c, m, n, k, 1, peers, s);
    case 4: return launch_cfg<QT, T, MXC, 1, Q6 ? 3 : 4>(a, b, bias, c, m, n, k, 2, peers, s);
    default: return RC_RANGE;
  }
}

template <int QT, typename T>
static int launch_q(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, int config, const PeerOut& peers,
                    cudaStream_t s) {
  if (m == 1) return launch_m<QT, T, 1>(a, b, bias, c, m, n, k, config, peers, s);
  if (m == 2) return launch_m<QT, T, 2>(a, b, bias, c, m, n, k, config, peers, s);
  if (m <= 4) return launch_m<QT, T, 4>(a, b, bias, c, m, n, k, config, peers, s);
  return launch_m<QT, T, 8>(a, b, bias, c, m, n, k, config, peers, s);
}

}  // namespace stream

bool gemv_stream_supports(int qtype, int dtype, int m, int n, int k) {
  (void)n;
  if (!(dtype == DINO_BF16 || dtype == DINO_F16) || m < 1 || m > 8) return false;
  if (qtype == QTYPE_Q4_K || qtype == QTYPE_Q5_K) return k % 256 == 0;      // 144 / 176-byte blocks: rows are always 16-byte multiples
  if (qtype == QTYPE_Q6_K) return k % 2048 == 0;      // 210-byte blocks: row pieces start on 16-byte boundaries only then
  // the further types: whole 256-weight groups and weight rows that are multiples of 16 bytes (bulk-copy sources)
  int sb_bytes = 0;
  switch (qtype) {
    case QTYPE_Q4_0: sb_bytes = 8 * 18; break;
    case QTYPE_Q2_K: sb_bytes = 84; break;
    case QTYPE_Q3_K: sb_bytes = 110; break;
    case QTYPE_MXFP4: sb_bytes = 8 * 17; break;
    case QTYPE_NVFP4: sb_bytes = 4 * 36; break;
    default: return false;
  }
  return k % 256 == 0 && (int64_t(k / 256) * sb_bytes) % 16 == 0;
}
int gemv_stream_configs() { return stream::kStreamConfigs; }

// peers: extra destinations of the result / gated epilogue (null = none); config: tuning configuration, 0 = default.
int gemm_rcr_stream_peers(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k, int config,
                          const PeerOut* peer_out, cudaStream_t s) {
  const PeerOut peers = peer_out != nullptr ? *peer_out : no_peers();
  if (int rc = check_gemm_args(a, b, c, qtype, dtype, m, n, k)) return rc;
  if (dtype == DINO_F32) return RC_DTYPE;
  if (m > 8) return RC_RANGE;
  if (qtype == QTYPE_Q8_0) return RC_QTYPE;
  if (!gemv_stream_supports(qtype, dtype, m, n, k)) return RC_ALIGN;
  if ((reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(a)) & 15) return RC_ALIGN;   // bulk-copy sources, vector loads
#define B200_STREAM_QTYPE(QT)                                                                                        \
  if (qtype == QT)                                                                                                    \
    return dtype == DINO_BF16 ? stream::launch_q<QT, __nv_bfloat16>(a, b, bias, c, m, n, k, config, peers, s)        \
                              : stream::launch_q<QT, __half>(a, b, bias, c, m, n, k, config, peers, s);
  B200_STREAM_QTYPE(QTYPE_Q6_K)
  B200_STREAM_QTYPE(QTYPE_Q4_0)
  B200_STREAM_QTYPE(QTYPE_Q5_K)
  B200_STREAM_QTYPE(QTYPE_Q2_K)
  B200_STREAM_QTYPE(QTYPE_Q3_K)
  B200_STREAM_QTYPE(QTYPE_MXFP4)
  B200_STREAM_QTYPE(QTYPE_NVFP4)
#undef B200_STREAM_QTYPE
  return dtype == DINO_BF16 ? stream::launch_q<QTYPE_Q4_K, __nv_bfloat16>(a, b, bias, c, m, n, k, config, peers, s)
                            : stream::launch_q<QTYPE_Q4_K, __half>(a, b, bias, c, m, n, k, config, peers, s);
}

int gemm_rcr_stream(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k, int config,
                    cudaStream_t s) {
  return gemm_rcr_stream_peers(a, b, bias, c, qtype, dtype, m, n, k, config, nullptr, s);
}

// Reads (and clears) the stream kernels' status word of the current device.
int stream_device_status() {
  int* status = stream::stream_status_ptr();
  int value = 0;
  if (status == nullptr) return -1;
  if (cudaMemcpy(&value, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (value != 0) {
    // a launch that gave up may have left partial-tile flags raised: lower them with the word
    cudaMemset(status, 0, sizeof(int));
    int dev = -1;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(stream::g_scratch_mutex);
    for (auto& entry : stream::g_scratch)
      if (entry.first.dev == dev && entry.second.flags != nullptr) cudaMemset(entry.second.flags, 0, size_t(stream::kMaxCtas) * sizeof(int));
  }
  return value;
}

}  // namespace b200gguf
