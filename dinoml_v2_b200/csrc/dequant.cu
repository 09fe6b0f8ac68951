// Standalone GGUF dequantize kernel: packed blocks -> dense f32 / f16 / bf16, bit-exact.
//
// Replaces the un-vendored libgguf device entry the reference's generated module declares at
// src/dinoml/templates/gpu_module.cu.j2:35-42 and calls from src/dinoml/lowering/ops/gemm.py:745,
// keeping its name and argument list so the generated launch text links unchanged.
//
// HBM-bound and write-dominated (Q4_K -> f32 writes 7.1 bytes per byte read).  Every packed byte is loaded once:
//   Q4_K: a thread owns 8 quant bytes = the low nibbles (8 weights of sub-block 2g) and the high nibbles (8 weights
//         of sub-block 2g+1) of one 64-weight group; 16 threads per block, the 16-byte header is one broadcast load;
//   Q6_K: a thread owns 8 positions l of one 128-weight half: 8 ql bytes, the 8 ql bytes 32 further, 8 qh bytes ->
//         four runs of 8 weights (one per quad); 8 threads per block;
//   Q8_0: a thread owns 8 consecutive weights.
//   the six further types: see dequant_items_kernel below.
// Decoding uses explicitly rounded fp32 operations (bit-exact), and each run of 8 outputs is one 32-byte (f32) or
// 16-byte (f16 / bf16) streaming store.  Float outputs (write bound) keep the simpler one-unit-per-thread kernel, which
// measured faster there (Q4_K -> f32 4.77 vs 4.35 TB/s); 16-bit outputs gain 8 % (Q4_K) to 35 % (Q6_K).
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

// Q8_0 and every float output: total_units = rows * n_per_row / 8.  Units are numbered in output order, so unit u
// covers outputs [8u, 8u+8) and lives in block u / (kBlock/8).
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

// Q4_K: item = (block, 64-weight group g, 8-byte piece p of the group's 32 quant bytes); 16 items per block.
// Formula per weight: (d * sc) * q - (dmin * m), each product / difference rounded (as decode8<QTYPE_Q4_K>).
template <typename T>
__global__ void __launch_bounds__(kDequantThreads)
dequant_q4k_kernel(const uint8_t* __restrict__ in, T* __restrict__ out, int64_t total_items) {
  const int64_t base = (int64_t(blockIdx.x) * 2) * kDequantThreads + threadIdx.x;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int64_t it = base + int64_t(i) * kDequantThreads;
    if (it >= total_items) continue;
    const int64_t blk = it >> 4;
    const int g = int(it & 15) >> 2, piece = int(it & 3);
    const uint8_t* b = in + blk * 144;                     // 4-byte aligned (checked by the launcher)
    const uint32_t* hdr = reinterpret_cast<const uint32_t*>(b);
    const uint32_t dd = __ldg(hdr), s0 = __ldg(hdr + 1), s1 = __ldg(hdr + 2), s2 = __ldg(hdr + 3);
    const float d = half_bits_to_float(uint16_t(dd & 0xffffu)), dmin = half_bits_to_float(uint16_t(dd >> 16));
    // 6-bit (scale, min) of sub-blocks 2g (low nibbles) and 2g+1 (high nibbles): bytes j, j+4 for j < 4, split fields after
    int sc[2], mn[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int j = 2 * g + h;
      if (j < 4) {
        sc[h] = int(s0 >> (8 * j)) & 63;
        mn[h] = int(s1 >> (8 * j)) & 63;
      } else {
        sc[h] = (int(s2 >> (8 * (j - 4))) & 0x0f) | ((int(s0 >> (8 * (j - 4))) >> 6 & 3) << 4);
        mn[h] = (int(s2 >> (8 * (j - 4))) >> 4 & 0x0f) | ((int(s1 >> (8 * (j - 4))) >> 6 & 3) << 4);
      }
    }
    const uint32_t* qp = reinterpret_cast<const uint32_t*>(b + 16 + 32 * g + 8 * piece);
    const uint2 q = make_uint2(__ldg(qp), __ldg(qp + 1));
    T* dst = out + blk * 256 + 64 * g + 8 * piece;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float ds = __fmul_rn(d, float(sc[h])), dm = __fmul_rn(dmin, float(mn[h]));
      const uint32_t q0 = q.x >> (4 * h), q1 = q.y >> (4 * h);
      float w[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        w[e] = __fsub_rn(__fmul_rn(ds, float((q0 >> (8 * e)) & 0x0f)), dm);
        w[4 + e] = __fsub_rn(__fmul_rn(ds, float((q1 >> (8 * e)) & 0x0f)), dm);
      }
      Pack8<T>::store(dst + 32 * h, w);
    }
  }
}

// Q6_K: item = (block, 128-weight half hb, 8 positions l0..l0+7); 8 items per block.  Weight 128*hb + 32*quad + l is
// (d * scale[8*hb + 2*quad + l/16]) * (q - 32) with q = nibble of ql | two bits of qh (as decode8<QTYPE_Q6_K>).
template <typename T>
__global__ void __launch_bounds__(kDequantThreads)
dequant_q6k_kernel(const uint8_t* __restrict__ in, T* __restrict__ out, int64_t total_items) {
  const int64_t base = (int64_t(blockIdx.x) * 2) * kDequantThreads + threadIdx.x;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int64_t it = base + int64_t(i) * kDequantThreads;
    if (it >= total_items) continue;
    const int64_t blk = it >> 3;
    const int hb = int(it & 7) >> 2, l0 = 8 * int(it & 3);
    const uint8_t* b = in + blk * 210;                     // 2-byte aligned
    const float d = half_bits_to_float(uint16_t(ld_u16(b + 208)));
    const uint32_t la[2] = {ld_u32_a2(b + 64 * hb + l0), ld_u32_a2(b + 64 * hb + l0 + 4)};
    const uint32_t lb[2] = {ld_u32_a2(b + 64 * hb + 32 + l0), ld_u32_a2(b + 64 * hb + 32 + l0 + 4)};
    const uint32_t hh[2] = {ld_u32_a2(b + 128 + 32 * hb + l0), ld_u32_a2(b + 128 + 32 * hb + l0 + 4)};
    const int8_t* scales = reinterpret_cast<const int8_t*>(b + 192) + 8 * hb + (l0 >> 4);
    T* dst = out + blk * 256 + 128 * hb + l0;
#pragma unroll
    for (int quad = 0; quad < 4; ++quad) {
      const float ds = __fmul_rn(d, float(int(scales[2 * quad])));
      float w[8];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t l4 = ((quad & 1) ? lb[h] : la[h]) >> ((quad & 2) ? 4 : 0);
        const uint32_t h4 = hh[h] >> (2 * quad);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int qv = int(((l4 >> (8 * e)) & 0x0f) | (((h4 >> (8 * e)) & 0x03) << 4)) - 32;
          w[4 * h + e] = __fmul_rn(ds, float(qv));
        }
      }
      Pack8<T>::store(dst + 32 * quad, w);
    }
  }
}

// The six further types, 16-bit outputs: item = 8 consecutive packed bytes and every run of 8 weights they hold, so that each
// packed byte is loaded once (the one-unit-per-thread kernel loads a nibble byte twice, a Q2_K byte four times and a Q3_K
// mask byte eight times).  Arithmetic is decode8<QT>'s, operation for operation.
//   Q4_0 / MXFP4: item = (block, half p of its 16 bytes): low nibbles = weights 8p .., high nibbles = weights 16 + 8p ..
//   NVFP4:        item = (block, sub-block s): low nibbles = its first 8 weights, high nibbles = the other 8
//   Q5_K:         item = (block, 64-weight group g, piece of 8 bytes): as Q4_K, plus bits 2g, 2g+1 of 8 bytes of qh
//   Q2_K / Q3_K:  item = (block, half hb, 8 positions l0 ..): four runs (bit pairs j = 0..3) of 8 weights 32 apart
// A: alignment the launcher found for the packed buffer (blocks of these types are only 1-, 2- or 4-byte multiples).
template <int QT> struct ItemGeom;
template <> struct ItemGeom<QTYPE_Q4_0> { static constexpr int kItems = 2, kAlign = 2; };
template <> struct ItemGeom<QTYPE_MXFP4> { static constexpr int kItems = 2, kAlign = 1; };
template <> struct ItemGeom<QTYPE_NVFP4> { static constexpr int kItems = 4, kAlign = 4; };
template <> struct ItemGeom<QTYPE_Q5_K> { static constexpr int kItems = 16, kAlign = 4; };
template <> struct ItemGeom<QTYPE_Q2_K> { static constexpr int kItems = 8, kAlign = 4; };
template <> struct ItemGeom<QTYPE_Q3_K> { static constexpr int kItems = 8, kAlign = 2; };
template <int QT> constexpr bool has_item_kernel() {
  return QT == QTYPE_Q4_0 || QT == QTYPE_MXFP4 || QT == QTYPE_NVFP4 || QT == QTYPE_Q5_K || QT == QTYPE_Q2_K || QT == QTYPE_Q3_K;
}

template <int A>
__device__ __forceinline__ uint2 ld8(const uint8_t* p) {      // 8 bytes at an A-byte aligned address
  if (A >= 4) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(p);
    return make_uint2(__ldg(w), __ldg(w + 1));
  }
  if (A == 2) return make_uint2(ld_u32_a2(p), ld_u32_a2(p + 4));
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) { lo |= uint32_t(p[i]) << (8 * i); hi |= uint32_t(p[4 + i]) << (8 * i); }
  return make_uint2(lo, hi);
}
__device__ __forceinline__ uint32_t byte_of(const uint2& q, int e) { return ((e < 4 ? q.x : q.y) >> (8 * (e & 3))) & 0xffu; }

template <int QT, typename T, int A>
__global__ void __launch_bounds__(kDequantThreads)
dequant_items_kernel(const uint8_t* __restrict__ in, T* __restrict__ out, int64_t total_items) {
  constexpr int kBytes = QTraits<QT>::kBytes, kBlock = QTraits<QT>::kBlock;
  const int64_t base = (int64_t(blockIdx.x) * 2) * kDequantThreads + threadIdx.x;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int64_t it = base + int64_t(i) * kDequantThreads;
    if (it >= total_items) continue;
    const int64_t blk = it / ItemGeom<QT>::kItems;
    const int item = int(it - blk * ItemGeom<QT>::kItems);
    const uint8_t* b = in + blk * kBytes;
    T* dst = out + blk * kBlock;
    float w[8];
    if constexpr (QT == QTYPE_Q4_0 || QT == QTYPE_MXFP4) {
      const float d = QT == QTYPE_Q4_0 ? half_at(b) : e8m0_half(b[0]);
      const uint2 q = ld8<A>(b + (kBytes - 16) + 8 * item);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t nib = (byte_of(q, e) >> (4 * h)) & 0x0fu;
          w[e] = QT == QTYPE_Q4_0 ? __fmul_rn(d, float(int(nib) - 8)) : __fmul_rn(d, float(fp4_code_value(nib)));
        }
        Pack8<T>::store(dst + 8 * item + 16 * h, w);
      }
    } else if constexpr (QT == QTYPE_NVFP4) {
      const float d = ue4m3_half(b[item]);
      const uint2 q = ld8<A>(b + 4 + 8 * item);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = __fmul_rn(d, float(fp4_code_value((byte_of(q, e) >> (4 * h)) & 0x0fu)));
        Pack8<T>::store(dst + 16 * item + 8 * h, w);
      }
    } else if constexpr (QT == QTYPE_Q5_K) {
      const int g = item >> 2, piece = item & 3;
      const uint2 q = ld8<A>(b + 48 + 32 * g + 8 * piece), qh = ld8<A>(b + 16 + 8 * piece);
      // the 16-byte header (d, dmin, 12 bytes of 6-bit scales and mins) as four words where the buffer is word aligned
      const uint2 h01 = ld8<A>(b), h23 = ld8<A>(b + 8);
      const float d = half_bits_to_float(uint16_t(h01.x & 0xffffu)), dmin = half_bits_to_float(uint16_t(h01.x >> 16));
      const uint32_t s0 = h01.y, s1 = h23.x, s2 = h23.y;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int j = 2 * g + h;
        int sc, mn;
        if (j < 4) {
          sc = int(s0 >> (8 * j)) & 63;
          mn = int(s1 >> (8 * j)) & 63;
        } else {
          sc = (int(s2 >> (8 * (j - 4))) & 0x0f) | ((int(s0 >> (8 * (j - 4))) >> 6 & 3) << 4);
          mn = (int(s2 >> (8 * (j - 4))) >> 4 & 0x0f) | ((int(s1 >> (8 * (j - 4))) >> 6 & 3) << 4);
        }
        const float ds = __fmul_rn(d, float(sc)), dm = __fmul_rn(dmin, float(mn));
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int qv = int((byte_of(q, e) >> (4 * h)) & 0x0fu) + (((byte_of(qh, e) >> (2 * g + h)) & 1u) ? 16 : 0);
          w[e] = __fsub_rn(__fmul_rn(ds, float(qv)), dm);
        }
        Pack8<T>::store(dst + 64 * g + 32 * h + 8 * piece, w);
      }
    } else {
      const int hb = item >> 2, l0 = 8 * (item & 3);
      constexpr int kQs = QT == QTYPE_Q2_K ? 16 : 32;
      const uint2 q = ld8<A>(b + kQs + 32 * hb + l0);
      uint2 hm = make_uint2(0u, 0u);
      if constexpr (QT == QTYPE_Q3_K) hm = ld8<A>(b + l0);
      const float d = half_at(b + (QT == QTYPE_Q2_K ? 80 : 108));
      const float dmin = QT == QTYPE_Q2_K ? half_at(b + 82) : 0.f;
      uint2 s01 = make_uint2(0u, 0u);          // Q3_K: the 12 scale bytes in three words (the third in s2)
      uint32_t s2 = 0u;
      if constexpr (QT == QTYPE_Q3_K) {
        s01 = ld8<A>(b + 96);
        s2 = A >= 2 ? ld_u32_a2(b + 104) : (uint32_t(b[104]) | (uint32_t(b[105]) << 8) | (uint32_t(b[106]) << 16) | (uint32_t(b[107]) << 24));
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int is = 8 * hb + 2 * j + (l0 >= 16 ? 1 : 0);
        if constexpr (QT == QTYPE_Q2_K) {
          const uint32_t scale = b[is];
          const float ds = __fmul_rn(d, float(scale & 0x0fu)), dm = __fmul_rn(dmin, float(scale >> 4));
#pragma unroll
          for (int e = 0; e < 8; ++e) w[e] = __fsub_rn(__fmul_rn(ds, float(int(byte_of(q, e) >> (2 * j)) & 3)), dm);
        } else {
          // 6-bit scale `is` = 4*qd + i4: low nibble in byte is % 8 (its high half for is >= 8), two high bits in byte 8 + i4 at bit 2*qd
          const int i4 = is & 3, qd = is >> 2;
          const uint32_t low = (((qd & 1) ? s01.y : s01.x) >> (8 * i4 + 4 * (qd >> 1))) & 0x0fu;
          const uint32_t high = (s2 >> (8 * i4 + 2 * qd)) & 0x03u;
          const float ds = __fmul_rn(d, float(int(low | (high << 4)) - 32));
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int low = int(byte_of(q, e) >> (2 * j)) & 3;
            w[e] = __fmul_rn(ds, float(low - (((byte_of(hm, e) >> (4 * hb + j)) & 1u) ? 0 : 4)));
          }
        }
        Pack8<T>::store(dst + 128 * hb + 32 * j + l0, w);
      }
    }
  }
}

template <int QT, typename T>
static int launch_dequant(const void* in, void* out, int64_t rows, int64_t n_per_row, cudaStream_t stream) {
  const int64_t weights = rows * n_per_row;
  // 16-bit outputs: the every-byte-once kernels; float outputs are write bound and measured faster with one 8-output
  // unit per thread (a warp then writes 1 KiB contiguous per pair of store instructions)
  if ((QT == QTYPE_Q4_K || QT == QTYPE_Q6_K) && sizeof(T) == 2) {
    const int64_t items = QT == QTYPE_Q4_K ? weights / 16 : weights / 32;
    const int64_t per_cta = int64_t(kDequantThreads) * 2;
    const int64_t grid = (items + per_cta - 1) / per_cta;
    if (grid > 0x7fffffffLL) return RC_RANGE;
    if (QT == QTYPE_Q4_K)
      dequant_q4k_kernel<T><<<dim3(unsigned(grid)), kDequantThreads, 0, stream>>>(static_cast<const uint8_t*>(in), static_cast<T*>(out), items);
    else
      dequant_q6k_kernel<T><<<dim3(unsigned(grid)), kDequantThreads, 0, stream>>>(static_cast<const uint8_t*>(in), static_cast<T*>(out), items);
    return cudaGetLastError() == cudaSuccess ? RC_OK : RC_LAUNCH;
  }
  if constexpr (has_item_kernel<QT>() && sizeof(T) == 2) {
    const int64_t items = weights / QTraits<QT>::kBlock * ItemGeom<QT>::kItems;
    const int64_t per_cta = int64_t(kDequantThreads) * 2;
    const int64_t grid = (items + per_cta - 1) / per_cta;
    if (grid > 0x7fffffffLL) return RC_RANGE;
    const uint8_t* src = static_cast<const uint8_t*>(in);
    // word loads where the packed buffer allows them (these types accept any byte address), byte loads otherwise
    if (ItemGeom<QT>::kAlign > 1 && reinterpret_cast<uintptr_t>(in) % ItemGeom<QT>::kAlign == 0)
      dequant_items_kernel<QT, T, ItemGeom<QT>::kAlign><<<dim3(unsigned(grid)), kDequantThreads, 0, stream>>>(src, static_cast<T*>(out), items);
    else
      dequant_items_kernel<QT, T, 1><<<dim3(unsigned(grid)), kDequantThreads, 0, stream>>>(src, static_cast<T*>(out), items);
    return cudaGetLastError() == cudaSuccess ? RC_OK : RC_LAUNCH;
  }
  const int64_t total_units = weights / 8;
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
  if ((in_a & uintptr_t(qtype_alignment(qtype) - 1)) || (out_a & 15)) return RC_ALIGN;
  switch (qtype) {
    case QTYPE_Q8_0: return launch_dequant_dtype<QTYPE_Q8_0>(dev_in, dev_out, rows, n_per_row, output_dtype, stream);
    case QTYPE_Q4_K: return launch_dequant_dtype<QTYPE_Q4_K>(dev_in, dev_out, rows, n_per_row, output_dtype, stream);
    case QTYPE_Q6_K: return launch_dequant_dtype<QTYPE_Q6_K>(dev_in, dev_out, rows, n_per_row, output_dtype, stream);
    case QTYPE_Q4_0: return launch_dequant_dtype<QTYPE_Q4_0>(dev_in, dev_out, rows, n_per_row, output_dtype, stream);
    case QTYPE_Q5_K: return launch_dequant_dtype<QTYPE_Q5_K>(dev_in, dev_out, rows, n_per_row, output_dtype, stream);
    case QTYPE_Q2_K: return launch_dequant_dtype<QTYPE_Q2_K>(dev_in, dev_out, rows, n_per_row, output_dtype, stream);
    case QTYPE_Q3_K: return launch_dequant_dtype<QTYPE_Q3_K>(dev_in, dev_out, rows, n_per_row, output_dtype, stream);
    case QTYPE_MXFP4: return launch_dequant_dtype<QTYPE_MXFP4>(dev_in, dev_out, rows, n_per_row, output_dtype, stream);
    case QTYPE_NVFP4: return launch_dequant_dtype<QTYPE_NVFP4>(dev_in, dev_out, rows, n_per_row, output_dtype, stream);
    default: return RC_QTYPE;
  }
}

}  // namespace b200gguf
