// Fused GGUF gemm_rcr, CUDA-core variant ("simt"): C[M,N] = A[M,K] * dequant(W[N,K])^T (+ bias).
//
// One warp per weight row; lanes stride over 8-wide K units, decode them exactly as the dequantizer
// does, and accumulate in fp32 with FMA; a shuffle tree finishes the row.  Every (activation, output)
// dtype and every M is supported, which makes this the reference-faithful fallback of the candidate
// family (the behavioural ancestor is the reference's one-wave-per-column prototype,
// kernels/rocm/src/ck_gguf_q8_gemm.hip:1168-1207) and the only variant that keeps fp32 activations
// un-rounded.  It reads W once per group of MT activation rows, so it is bandwidth-efficient only
// for M <= MT; the tensor-core variants take over elsewhere.
#include "gguf_common.cuh"

namespace b200gguf {

template <typename T> __device__ __forceinline__ void load8(const T* p, float (&x)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&x)[8]) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__half>(const __half* p, float (&x)[8]) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[8]) {
  const uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
  const uint32_t r[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { x[2 * i] = __uint_as_float(r[i] << 16); x[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u); }
}

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

constexpr int kSimtWarps = 8;

template <int QT, typename T, int MT>
__global__ void __launch_bounds__(kSimtWarps * 32)
gemm_rcr_simt_kernel(const T* __restrict__ a, const uint8_t* __restrict__ b, const T* __restrict__ bias,
                     T* __restrict__ c, int m, int n, int k) {
  constexpr int kUnitsPerBlock = QTraits<QT>::kBlock / 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * kSimtWarps + warp;
  const int m0 = blockIdx.y * MT;
  if (col >= n) return;
  const int64_t row_bytes = int64_t(k / QTraits<QT>::kBlock) * QTraits<QT>::kBytes;
  const uint8_t* wrow = b + int64_t(col) * row_bytes;
  float acc[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i) acc[i] = 0.f;
  const int units = k >> 3;
  for (int u = lane; u < units; u += 32) {
    const int blk = u / kUnitsPerBlock;
    const int kk0 = (u - blk * kUnitsPerBlock) * 8;
    float w[8];
    decode8<QT>(wrow + int64_t(blk) * QTraits<QT>::kBytes, kk0, w);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (m0 + i < m) {
        float x[8];
        load8<T>(a + int64_t(m0 + i) * k + int64_t(u) * 8, x);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i] = fmaf(x[j], w[j], acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MT; ++i) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], off);
  }
  if (lane == 0) {
    const float bv = bias != nullptr ? to_float<T>(bias[col]) : 0.f;
#pragma unroll
    for (int i = 0; i < MT; ++i)
      if (m0 + i < m) c[int64_t(m0 + i) * n + col] = from_float<T>(acc[i] + bv);
  }
}

template <int QT, typename T>
static int launch_simt_t(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, cudaStream_t s) {
  const dim3 block(kSimtWarps * 32);
  if (m == 1) {
    const dim3 grid((n + kSimtWarps - 1) / kSimtWarps, 1);
    gemm_rcr_simt_kernel<QT, T, 1><<<grid, block, 0, s>>>(static_cast<const T*>(a), static_cast<const uint8_t*>(b),
                                                          static_cast<const T*>(bias), static_cast<T*>(c), m, n, k);
  } else {
    const dim3 grid((n + kSimtWarps - 1) / kSimtWarps, (m + 3) / 4);
    if (grid.y > 65535) return RC_RANGE;
    gemm_rcr_simt_kernel<QT, T, 4><<<grid, block, 0, s>>>(static_cast<const T*>(a), static_cast<const uint8_t*>(b),
                                                          static_cast<const T*>(bias), static_cast<T*>(c), m, n, k);
  }
  return cudaGetLastError() == cudaSuccess ? RC_OK : RC_LAUNCH;
}

template <int QT>
static int launch_simt_q(const void* a, const void* b, const void* bias, void* c, int dtype, int m, int n, int k,
                         cudaStream_t s) {
  switch (dtype) {
    case DINO_F32: return launch_simt_t<QT, float>(a, b, bias, c, m, n, k, s);
    case DINO_F16: return launch_simt_t<QT, __half>(a, b, bias, c, m, n, k, s);
    case DINO_BF16: return launch_simt_t<QT, __nv_bfloat16>(a, b, bias, c, m, n, k, s);
    default: return RC_DTYPE;
  }
}

// Shared argument validation of every fused-gemm variant.
int check_gemm_args(const void* a, const void* b, const void* c, int qtype, int dtype, int m, int n, int k) {
  if (a == nullptr || b == nullptr || c == nullptr) return RC_NULL;
  if (m <= 0 || n <= 0 || k <= 0) return RC_DIMS;
  const int bs = qtype_block_size(qtype);
  if (bs == 0) return RC_QTYPE;
  if (k % bs) return RC_KBLOCK;
  if (dtype != DINO_F32 && dtype != DINO_F16 && dtype != DINO_BF16) return RC_DTYPE;
  const uintptr_t aa = reinterpret_cast<uintptr_t>(a), ba = reinterpret_cast<uintptr_t>(b);
  const int64_t row_bytes = int64_t(k / bs) * qtype_block_bytes(qtype);
  const uintptr_t wmask = uintptr_t(qtype_alignment(qtype) - 1);
  if ((aa & 15) || (ba & wmask) || (uintptr_t(row_bytes) & wmask)) return RC_ALIGN;
  return RC_OK;
}

int gemm_rcr_simt(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                  cudaStream_t s) {
  if (int rc = check_gemm_args(a, b, c, qtype, dtype, m, n, k)) return rc;
  switch (qtype) {
    case QTYPE_Q8_0: return launch_simt_q<QTYPE_Q8_0>(a, b, bias, c, dtype, m, n, k, s);
    case QTYPE_Q4_K: return launch_simt_q<QTYPE_Q4_K>(a, b, bias, c, dtype, m, n, k, s);
    case QTYPE_Q6_K: return launch_simt_q<QTYPE_Q6_K>(a, b, bias, c, dtype, m, n, k, s);
    case QTYPE_Q4_0: return launch_simt_q<QTYPE_Q4_0>(a, b, bias, c, dtype, m, n, k, s);
    case QTYPE_Q5_K: return launch_simt_q<QTYPE_Q5_K>(a, b, bias, c, dtype, m, n, k, s);
    case QTYPE_Q2_K: return launch_simt_q<QTYPE_Q2_K>(a, b, bias, c, dtype, m, n, k, s);
    case QTYPE_Q3_K: return launch_simt_q<QTYPE_Q3_K>(a, b, bias, c, dtype, m, n, k, s);
    case QTYPE_MXFP4: return launch_simt_q<QTYPE_MXFP4>(a, b, bias, c, dtype, m, n, k, s);
    case QTYPE_NVFP4: return launch_simt_q<QTYPE_NVFP4>(a, b, bias, c, dtype, m, n, k, s);
    default: return RC_QTYPE;
  }
}

}  // namespace b200gguf
