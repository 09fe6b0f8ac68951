// Shared device/host definitions for the GGUF quantized-linear kernels (sm_100a).
//
// Block layouts and decode arithmetic follow the reference's statements of them:
// kernels/rocm/src/ck_gguf_q8_gemm.hip:20-25,34-41,71-78 (structs), :143-155
// (6-bit scale/min unpack), :724-739 / :764-802 / :920-960 (per-element decode).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200gguf {

// ggml type ids, as stored in the reference's constant metadata (qtype_value).
enum : int { QTYPE_Q4_0 = 2, QTYPE_Q8_0 = 8, QTYPE_Q2_K = 10, QTYPE_Q3_K = 11, QTYPE_Q4_K = 12, QTYPE_Q5_K = 13, QTYPE_Q6_K = 14,
              QTYPE_MXFP4 = 39, QTYPE_NVFP4 = 40 };
// Dense dtype codes of the dequantizer ABI (0/1 are the reference's; 2 is an extension).
enum : int { OUT_F32 = 0, OUT_F16 = 1, OUT_BF16 = 2 };
// DinoDtype values of runtime ABI v7 (runtime/include/dinoml/abi.h:14-23).
enum : int { DINO_F16 = 1, DINO_F32 = 2, DINO_BF16 = 6 };

// Launcher return codes.  1..3 follow kernels/rocm/src/ck_gguf_q8_gemm.hip:1910-1918.
enum : int {
  RC_OK = 0,
  RC_NULL = 1,        // null pointer
  RC_DIMS = 2,        // non-positive dimension
  RC_KBLOCK = 3,      // k (n_per_row) not a multiple of the block size
  RC_LAUNCH = 4,      // CUDA launch failure
  RC_QTYPE = 5,       // unsupported quantization type
  RC_DTYPE = 6,       // unsupported activation/output dtype
  RC_ALIGN = 7,       // pointer / row pitch alignment not met for this variant
  RC_RANGE = 8,       // shape outside what this variant supports
  RC_DEVICE = 9,      // device-side bounded wait gave up (status word set)
};

struct __align__(2) BlockQ8_0 { uint16_t d; int8_t qs[32]; };
struct __align__(4) BlockQ4_K { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qs[128]; };
struct __align__(2) BlockQ6_K { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; };
static_assert(sizeof(BlockQ8_0) == 34, "Q8_0 block must be 34 bytes");
static_assert(sizeof(BlockQ4_K) == 144, "Q4_K block must be 144 bytes");
static_assert(sizeof(BlockQ6_K) == 210, "Q6_K block must be 210 bytes");

template <int QT> struct QTraits;
template <> struct QTraits<QTYPE_Q8_0> { static constexpr int kBlock = 32,  kBytes = 34;  using Block = BlockQ8_0; };
template <> struct QTraits<QTYPE_Q4_K> { static constexpr int kBlock = 256, kBytes = 144; using Block = BlockQ4_K; };
template <> struct QTraits<QTYPE_Q6_K> { static constexpr int kBlock = 256, kBytes = 210; using Block = BlockQ6_K; };
// The further layouts of the reference's fused prototype (kernels/rocm/src/ck_gguf_q8_gemm.hip:27-32, 43-69, 80-92); they are
// decoded with byte loads, so they carry no alignment requirement.
//   Q4_0:  u16 d; u8 qs[16]                                            18 B / 32 weights
//   Q5_K:  u16 d; u16 dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]       176 B / 256
//   Q2_K:  u8 scales[16]; u8 qs[64]; u16 d; u16 dmin                   84 B / 256
//   Q3_K:  u8 hmask[32]; u8 qs[64]; u8 scales[12]; u16 d               110 B / 256
//   MXFP4: u8 e; u8 qs[16]                                             17 B / 32
//   NVFP4: u8 d[4]; u8 qs[32]                                          36 B / 64
template <> struct QTraits<QTYPE_Q4_0> { static constexpr int kBlock = 32, kBytes = 18; };
template <> struct QTraits<QTYPE_Q5_K> { static constexpr int kBlock = 256, kBytes = 176; };
template <> struct QTraits<QTYPE_Q2_K> { static constexpr int kBlock = 256, kBytes = 84; };
template <> struct QTraits<QTYPE_Q3_K> { static constexpr int kBlock = 256, kBytes = 110; };
template <> struct QTraits<QTYPE_MXFP4> { static constexpr int kBlock = 32, kBytes = 17; };
template <> struct QTraits<QTYPE_NVFP4> { static constexpr int kBlock = 64, kBytes = 36; };

__host__ __device__ inline int qtype_block_size(int64_t qt) {
  switch (qt) {
    case QTYPE_Q8_0: case QTYPE_Q4_0: case QTYPE_MXFP4: return 32;
    case QTYPE_NVFP4: return 64;
    case QTYPE_Q2_K: case QTYPE_Q3_K: case QTYPE_Q4_K: case QTYPE_Q5_K: case QTYPE_Q6_K: return 256;
    default: return 0;
  }
}
__host__ __device__ inline int qtype_block_bytes(int64_t qt) {
  switch (qt) {
    case QTYPE_Q4_0: return 18;  case QTYPE_Q8_0: return 34;  case QTYPE_Q2_K: return 84;  case QTYPE_Q3_K: return 110;
    case QTYPE_Q4_K: return 144; case QTYPE_Q5_K: return 176; case QTYPE_Q6_K: return 210; case QTYPE_MXFP4: return 17;
    case QTYPE_NVFP4: return 36;
    default: return 0;
  }
}
// Address alignment the decoders need from the start of a weight buffer (and of every row).
__host__ __device__ inline int qtype_alignment(int64_t qt) {
  return qt == QTYPE_Q4_K ? 4 : (qt == QTYPE_Q8_0 || qt == QTYPE_Q6_K) ? 2 : 1;
}

#ifdef __CUDACC__
__device__ __forceinline__ float half_bits_to_float(uint16_t bits) {
  return __half2float(__ushort_as_half(bits));
}

// 16-bit / 32-bit loads from 2-byte aligned addresses (Q8_0 and Q6_K blocks are only 2-aligned).
__device__ __forceinline__ uint32_t ld_u16(const void* p) { return *reinterpret_cast<const uint16_t*>(p); }
__device__ __forceinline__ uint32_t ld_u32_a2(const void* p) {
  const uint16_t* h = reinterpret_cast<const uint16_t*>(p);
  return uint32_t(h[0]) | (uint32_t(h[1]) << 16);
}

// (scale, min) of Q4_K / Q5_K sub-block j (0..7) from the 12 packed bytes.
__device__ __forceinline__ void k4_scale_min(int j, const uint8_t* q, int& sc, int& mn) {
  if (j < 4) {
    sc = q[j] & 63;
    mn = q[j + 4] & 63;
  } else {
    sc = (q[j + 4] & 0x0f) | ((q[j - 4] >> 6) << 4);
    mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// Exact (bit-reproducible) decode of 8 consecutive weights kk0..kk0+7 (kk0 % 8 == 0) of one block.
// Every product / difference is an explicitly rounded fp32 operation (__fmul_rn / __fsub_rn are never
// contracted into FMA), which is what the reference's --fmad=false dequantizer build computes
// (CMakeLists.txt:1683,1698,1719): Q8_0 d*q ; Q4_K (d*sc)*q - (dmin*m) ; Q6_K (d*scale)*q.
template <int QT> __device__ __forceinline__ void decode8(const uint8_t* blk, int kk0, float (&w)[8]);

template <> __device__ __forceinline__ void decode8<QTYPE_Q8_0>(const uint8_t* blk, int kk0, float (&w)[8]) {
  const float d = half_bits_to_float(ld_u16(blk));
  const uint32_t lo = ld_u32_a2(blk + 2 + kk0), hi = ld_u32_a2(blk + 2 + kk0 + 4);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    w[i] = __fmul_rn(d, float(int(int8_t(lo >> (8 * i)))));
    w[4 + i] = __fmul_rn(d, float(int(int8_t(hi >> (8 * i)))));
  }
}

template <> __device__ __forceinline__ void decode8<QTYPE_Q4_K>(const uint8_t* blk, int kk0, float (&w)[8]) {
  const BlockQ4_K* b = reinterpret_cast<const BlockQ4_K*>(blk);
  const int group64 = kk0 >> 6, local64 = kk0 & 63;
  const int high = local64 >= 32;
  const int local32 = local64 & 31;
  int sc, mn;
  k4_scale_min(group64 * 2 + high, b->scales, sc, mn);
  const float ds = __fmul_rn(half_bits_to_float(b->d), float(sc));
  const float dm = __fmul_rn(half_bits_to_float(b->dmin), float(mn));
  const uint32_t* qp = reinterpret_cast<const uint32_t*>(b->qs + group64 * 32 + local32);
  const uint32_t q0 = qp[0] >> (4 * high), q1 = qp[1] >> (4 * high);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    w[i] = __fsub_rn(__fmul_rn(ds, float((q0 >> (8 * i)) & 0x0f)), dm);
    w[4 + i] = __fsub_rn(__fmul_rn(ds, float((q1 >> (8 * i)) & 0x0f)), dm);
  }
}

template <> __device__ __forceinline__ void decode8<QTYPE_Q6_K>(const uint8_t* blk, int kk0, float (&w)[8]) {
  const BlockQ6_K* b = reinterpret_cast<const BlockQ6_K*>(blk);
  const int half_block = kk0 >> 7, local128 = kk0 & 127;
  const int quad = local128 >> 5, local32 = local128 & 31;
  const int ql_index = half_block * 64 + ((quad & 1) ? 32 : 0) + local32;
  const int qh_index = half_block * 32 + local32;
  const int scale_index = half_block * 8 + 2 * quad + (local32 >= 16 ? 1 : 0);
  const float ds = __fmul_rn(half_bits_to_float(ld_u16(&b->d)), float(int(b->scales[scale_index])));
  const int lsh = quad >= 2 ? 4 : 0, hsh = 2 * quad;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t l4 = ld_u32_a2(b->ql + ql_index + 4 * h) >> lsh;
    const uint32_t h4 = ld_u32_a2(b->qh + qh_index + 4 * h) >> hsh;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int q = int(((l4 >> (8 * i)) & 0x0f) | (((h4 >> (8 * i)) & 0x03) << 4)) - 32;
      w[4 * h + i] = __fmul_rn(ds, float(q));
    }
  }
}
// ---- the further types.  Field order and arithmetic follow the reference's host statements of them,
// tools/bench_ck_gguf_q8_gemm.hip:2038-2076 (Q3_K scale, e8m0 / ue4m3 scales, FP4 values) and :2084-2189 (values); every
// product and difference is an explicitly rounded fp32 operation, as for the three types above.
__device__ __forceinline__ float half_at(const uint8_t* p) { return half_bits_to_float(uint16_t(p[0] | (uint32_t(p[1]) << 8))); }
// twice the value of an FP4 (e2m1) code, as an integer: {0, 1, 2, 3, 4, 6, 8, 12} with bit 3 the sign
__device__ __forceinline__ int fp4_code_value(uint32_t q) {
  const int mag = int((0xC8643210u >> (4 * (q & 7u))) & 0xfu);
  return (q & 8u) ? -mag : mag;
}
// half of 2^(x - 127) (e8m0 scale of an MXFP4 block)
__device__ __forceinline__ float e8m0_half(uint32_t x) { return __uint_as_float(x < 2 ? (0x00200000u << x) : ((x - 1) << 23)); }
// half of an unsigned e4m3 scale (NVFP4 sub-block); 0x00 and 0x7f decode to 0
__device__ __forceinline__ float ue4m3_half(uint32_t x) {
  if (x == 0 || x == 0x7f) return 0.f;
  const uint32_t exp = (x >> 3) & 0x0f, man = x & 7;
  const float raw = exp == 0 ? __fmul_rn(float(man), __uint_as_float((127u - 9u) << 23))
                             : __fmul_rn(__fadd_rn(1.0f, __fmul_rn(float(man), 0.125f)), __uint_as_float((127u + exp - 7u) << 23));
  return __fmul_rn(0.5f, raw);
}

template <> __device__ __forceinline__ void decode8<QTYPE_Q4_0>(const uint8_t* blk, int kk0, float (&w)[8]) {
  const float d = half_at(blk);
  const int high = kk0 >= 16;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t packed = blk[2 + (kk0 & 15) + i];
    w[i] = __fmul_rn(d, float(int(high ? packed >> 4 : packed & 0x0f) - 8));
  }
}

template <> __device__ __forceinline__ void decode8<QTYPE_Q5_K>(const uint8_t* blk, int kk0, float (&w)[8]) {
  const int group64 = kk0 >> 6, high = (kk0 & 63) >= 32, local32 = kk0 & 31;
  int sc, mn;
  k4_scale_min(group64 * 2 + high, blk + 4, sc, mn);
  const float ds = __fmul_rn(half_at(blk), float(sc));
  const float dm = __fmul_rn(half_at(blk + 2), float(mn));
  const uint32_t bit = (high ? 2u : 1u) << (2 * group64);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t packed = blk[48 + group64 * 32 + local32 + i];
    const int q = int(high ? packed >> 4 : packed & 0x0f) + ((blk[16 + local32 + i] & bit) ? 16 : 0);
    w[i] = __fsub_rn(__fmul_rn(ds, float(q)), dm);
  }
}

template <> __device__ __forceinline__ void decode8<QTYPE_Q2_K>(const uint8_t* blk, int kk0, float (&w)[8]) {
  const int half_block = kk0 >> 7, j = (kk0 & 127) >> 5, local32 = kk0 & 31;
  const uint32_t scale = blk[half_block * 8 + 2 * j + (local32 >= 16 ? 1 : 0)];
  const float ds = __fmul_rn(half_at(blk + 80), float(scale & 0x0f));
  const float dm = __fmul_rn(half_at(blk + 82), float(scale >> 4));
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int q = int(blk[16 + half_block * 32 + local32 + i] >> (2 * j)) & 3;
    w[i] = __fsub_rn(__fmul_rn(ds, float(q)), dm);
  }
}

__device__ __forceinline__ int q3k_scale(const uint8_t* scales, int is) {
  if (is < 4) return (scales[is] & 0x0f) | ((scales[is + 8] & 0x03) << 4);
  if (is < 8) return (scales[is] & 0x0f) | (((scales[is + 4] >> 2) & 0x03) << 4);
  if (is < 12) return (scales[is - 8] >> 4) | (((scales[is] >> 4) & 0x03) << 4);
  return (scales[is - 8] >> 4) | (((scales[is - 4] >> 6) & 0x03) << 4);
}
template <> __device__ __forceinline__ void decode8<QTYPE_Q3_K>(const uint8_t* blk, int kk0, float (&w)[8]) {
  const int half_block = kk0 >> 7, j = (kk0 & 127) >> 5, local32 = kk0 & 31;
  const int scale = q3k_scale(blk + 96, 8 * half_block + 2 * j + (local32 >= 16 ? 1 : 0)) - 32;
  const float ds = __fmul_rn(half_at(blk + 108), float(scale));
  const uint32_t mask = 1u << (4 * half_block + j);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int low = int(blk[32 + half_block * 32 + local32 + i] >> (2 * j)) & 3;
    w[i] = __fmul_rn(ds, float(low - ((blk[local32 + i] & mask) ? 0 : 4)));
  }
}

template <> __device__ __forceinline__ void decode8<QTYPE_MXFP4>(const uint8_t* blk, int kk0, float (&w)[8]) {
  const float e = e8m0_half(blk[0]);
  const int high = kk0 >= 16;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t packed = blk[1 + (kk0 & 15) + i];
    w[i] = __fmul_rn(e, float(fp4_code_value(high ? packed >> 4 : packed & 0x0f)));
  }
}

template <> __device__ __forceinline__ void decode8<QTYPE_NVFP4>(const uint8_t* blk, int kk0, float (&w)[8]) {
  const int sub = kk0 >> 4, high = (kk0 & 15) >= 8;
  const float d = ue4m3_half(blk[sub]);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t packed = blk[4 + sub * 8 + i];
    w[i] = __fmul_rn(d, float(fp4_code_value(high ? packed >> 4 : packed & 0x0f)));
  }
}
#endif  // __CUDACC__

}  // namespace b200gguf
