// Standalone GGUF dequantize kernel: packed blocks -> dense f32 / f16 / bf16, bit-exact.
//
// Replaces the un-vendored libgguf device entry the reference's generated module declares at
// src/dinoml/templates/gpu_module.cu.j2:35-42 and calls from src/dinoml/lowering/ops/gemm.py:745,
// keeping its name and argument list so the generated launch text links unchanged.
//
// HBM-bound and write-dominated (Q4_K -> f32 writes 7.1 bytes per byte read).  One thread owns one
// "unit" of 8 consecutive outputs: it reads the few packed bytes that unit needs (the block header
// is shared by the 32 units of a K-quant block and is served by L1), decodes with explicitly rounded
// fp32 operations, and issues one 32-byte (f32) or 16-byte (f16/bf16) store.  Consecutive threads own
// consecutive units, so a warp writes 1 KiB (f32) contiguous per store instruction.
#include "gguf_common.cuh"

namespace b200gguf {

template <typename T> struct Pack8;
template <> struct Pack8<float> {
  static __device__ __forceinline__ void store(float* dst, const float (&w)[8]) {
    float4* p = reinterpret_cast<float4*>(dst);
    __stcs(p, make_float4(w[0], w[1], w[2], w[3]));
    __stcs(p + 1, make_float4(w[4], w[5], w[6], w[7]));
  }
};
template <> struct Pack8<__half> {
  static __device__ __forceinline__ void store(__half* dst, const float (&w)[8]) {
    uint4 v;
    __half2 h;
    h = __floats2half2_rn(w[0], w[1]); v.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(w[2], w[3]); v.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(w[4], w[5]); v.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2half2_rn(w[6], w[7]); v.w = *reinterpret_cast<uint32_t*>(&h);
    __stcs(reinterpret_cast<uint4*>(dst), v);
  }
};
template <> struct Pack8<__nv_bfloat16> {
  static __device__ __forceinline__ void store(__nv_bfloat16* dst, const float (&w)[8]) {
    uint4 v;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(w[0], w[1]); v.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(w[2], w[3]); v.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(w[4], w[5]); v.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(w[6], w[7]); v.w = *reinterpret_cast<uint32_t*>(&h);
    __stcs(reinterpret_cast<uint4*>(dst), v);
  }
};

constexpr int kDequantThreads = 256;
constexpr int kUnitsPerThread = 4;

// total_units = rows * n_per_row / 8.  Units are numbered in output order, so unit u covers
// outputs [8u, 8u+8) and lives in block u / (kBlock/8).
template <int QT, typename T>
__global__ void __launch_bounds__(kDequantThreads)
dequant_rows_kernel(const uint8_t* __restrict__ in, T* __restrict__ out, int64_t total_units) {
  constexpr int kUnitsPerBlock = QTraits<QT>::kBlock / 8;
  const int64_t base = (int64_t(blockIdx.x) * kUnitsPerThread) * kDequantThreads + threadIdx.x;
#pragma unroll
  for (int i = 0; i < kUnitsPerThread; ++i) {
    const int64_t u = base + int64_t(i) * kDequantThreads;
    if (u < total_units) {
      const int64_t blk = u / kUnitsPerBlock;
      const int kk0 = int(u - blk * kUnitsPerBlock) * 8;
      float w[8];
      decode8<QT>(in + blk * QTraits<QT>::kBytes, kk0, w);
      Pack8<T>::store(out + u * 8, w);
    }
  }
}

template <int QT, typename T>
static int launch_dequant(const void* in, void* out, int64_t rows, int64_t n_per_row, cudaStream_t stream) {
  const int64_t total_units = rows * n_per_row / 8;
  const int64_t per_cta = int64_t(kDequantThreads) * kUnitsPerThread;
  const int64_t grid = (total_units + per_cta - 1) / per_cta;
  if (grid > 0x7fffffffLL) return RC_RANGE;
  dequant_rows_kernel<QT, T><<<dim3(unsigned(grid)), kDequantThreads, 0, stream>>>(
      static_cast<const uint8_t*>(in), static_cast<T*>(out), total_units);
  return cudaGetLastError() == cudaSuccess ? RC_OK : RC_LAUNCH;
}

template <int QT>
static int launch_dequant_dtype(const void* in, void* out, int64_t rows, int64_t n_per_row, int out_dtype,
                                cudaStream_t stream) {
  switch (out_dtype) {
    case OUT_F32: return launch_dequant<QT, float>(in, out, rows, n_per_row, stream);
    case OUT_F16: return launch_dequant<QT, __half>(in, out, rows, n_per_row, stream);
    case OUT_BF16: return launch_dequant<QT, __nv_bfloat16>(in, out, rows, n_per_row, stream);
    default: return RC_DTYPE;
  }
}

int dequantize_rows(const void* dev_in, int64_t qtype, int64_t rows, int64_t n_per_row, int output_dtype,
                    void* dev_out, cudaStream_t stream) {
  if (dev_in == nullptr || dev_out == nullptr) return RC_NULL;
  if (rows <= 0 || n_per_row <= 0) return RC_DIMS;
  const int bs = qtype_block_size(qtype);
  if (bs == 0) return RC_QTYPE;
  if (n_per_row % bs) return RC_KBLOCK;
  const uintptr_t in_a = reinterpret_cast<uintptr_t>(dev_in), out_a = reinterpret_cast<uintptr_t>(dev_out);
  if ((in_a & (qtype == QTYPE_Q4_K ? 3 : 1)) || (out_a & 15)) return RC_ALIGN;
  switch (qtype) {
    case QTYPE_Q8_0: return launch_dequant_dtype<QTYPE_Q8_0>(dev_in, dev_out, rows, n_per_row, output_dtype, stream);
    case QTYPE_Q4_K: return launch_dequant_dtype<QTYPE_Q4_K>(dev_in, dev_out, rows, n_per_row, output_dtype, stream);
    case QTYPE_Q6_K: return launch_dequant_dtype<QTYPE_Q6_K>(dev_in, dev_out, rows, n_per_row, output_dtype, stream);
    default: return RC_QTYPE;
  }
}

}  // namespace b200gguf
