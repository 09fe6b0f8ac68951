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
enum : int { QTYPE_Q8_0 = 8, QTYPE_Q4_K = 12, QTYPE_Q6_K = 14 };
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

__host__ __device__ inline int qtype_block_size(int64_t qt) {
  return qt == QTYPE_Q8_0 ? 32 : (qt == QTYPE_Q4_K || qt == QTYPE_Q6_K) ? 256 : 0;
}
__host__ __device__ inline int qtype_block_bytes(int64_t qt) {
  return qt == QTYPE_Q8_0 ? 34 : qt == QTYPE_Q4_K ? 144 : qt == QTYPE_Q6_K ? 210 : 0;
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

// (scale, min) of Q4_K sub-block j (0..7) from the 12 packed bytes.
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
#endif  // __CUDACC__

}  // namespace b200gguf
