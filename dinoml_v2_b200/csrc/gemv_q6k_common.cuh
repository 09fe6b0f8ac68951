// Q6_K arithmetic shared by the decode GEMV kernels (tile kernel gemv_q6k_mma.cu, persistent kernel gemv_stream.cu): one
// 256-weight super-block of 16 weight rows on one warp, from packed bytes in shared memory to scaled fp32 sums.
#pragma once
#include "gemv_mma_common.cuh"

namespace b200gguf {

constexpr int kQ6ScalePitch = 20;                        // floats per row of the scale scratch: 16 + 4 so that the 16-byte reads of 8 rows hit all banks

template <typename T> struct Q6Offset;
template <> struct Q6Offset<__nv_bfloat16> { static constexpr uint32_t kPair = 0x43204320u; };   // 160 = 128 + 32
template <> struct Q6Offset<__half> { static constexpr uint32_t kPair = 0x64206420u; };          // 1056 = 1024 + 32

template <typename T> struct Pair2;
template <> struct Pair2<__nv_bfloat16> { using V = __nv_bfloat162; };
template <> struct Pair2<__half> { using V = __half2; };

// (MAGIC + q) pair -> (q - 32) pair, exact.
template <typename T>
__device__ __forceinline__ uint32_t q6_center(uint32_t pair) {
  using V = typename Pair2<T>::V;
  const uint32_t off = Q6Offset<T>::kPair;
  const V v = __hsub2(*reinterpret_cast<const V*>(&pair), *reinterpret_cast<const V*>(&off));
  return *reinterpret_cast<const uint32_t*>(&v);
}

// 32-bit word at a shared-memory address that is 4-byte aligned (MODE 0), 2 bytes past alignment (MODE 1), or either,
// decided per address at run time (MODE 2: weight rows that are not 16-byte multiples put every row at its own phase).
enum : int { Q6_ALIGNED = 0, Q6_ODD = 1, Q6_RUNTIME = 2 };
template <int MODE>
__device__ __forceinline__ uint32_t lds_word(const uint8_t* p) {
  if (MODE == Q6_ALIGNED) return *reinterpret_cast<const uint32_t*>(p);
  if (MODE == Q6_ODD) {
    const uint32_t* q = reinterpret_cast<const uint32_t*>(p - 2);
    return __byte_perm(q[0], q[1], 0x5432);
  }
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  const uint32_t* q = reinterpret_cast<const uint32_t*>(a & ~uintptr_t(3));
  return __byte_perm(q[0], q[1], (a & 2) ? 0x5432u : 0x3210u);
}

// One super-block of 16 rows on one warp.  blk: the staged block of row lane/2 (this lane decodes half of its scales),
// b0 / b1: the staged blocks of rows lane/4 and lane/4 + 8 (this lane's MMA rows).
template <typename T, int NT, int MC, int ODD>
__device__ __forceinline__ void q6k_superblock(const uint8_t* blk, const uint8_t* b0, const uint8_t* b1, float (*sS)[kQ6ScalePitch],
                                               const T* const (&xrow)[NT], int sb, int lane, float (&res)[NT][4]) {
  using MT = MmaType<T>;
  const int g = lane >> 2, t = lane & 3;
  {   // lane pair (row = lane/2, half = lane%2): 8 int8 scales -> d * sc as floats in shared memory
    const int srow = lane >> 1, shalf = lane & 1;
    const float d = half_bits_to_float(*reinterpret_cast<const uint16_t*>(blk + 208));
    const uint32_t s0 = lds_word<ODD>(blk + 192 + 8 * shalf) ^ 0x80808080u;   // int8 + 128 as unsigned bytes
    const uint32_t s1 = lds_word<ODD>(blk + 196 + 8 * shalf) ^ 0x80808080u;
    float4 lo, hi;
    lo.x = d * (byte_to_float(s0, 0) - 128.f); lo.y = d * (byte_to_float(s0, 1) - 128.f);
    lo.z = d * (byte_to_float(s0, 2) - 128.f); lo.w = d * (byte_to_float(s0, 3) - 128.f);
    hi.x = d * (byte_to_float(s1, 0) - 128.f); hi.y = d * (byte_to_float(s1, 1) - 128.f);
    hi.z = d * (byte_to_float(s1, 2) - 128.f); hi.w = d * (byte_to_float(s1, 3) - 128.f);
    *reinterpret_cast<float4*>(&sS[srow][8 * shalf]) = lo;
    *reinterpret_cast<float4*>(&sS[srow][8 * shalf + 4]) = hi;
  }
  __syncwarp();
#pragma unroll
  for (int hb = 0; hb < 2; ++hb) {                   // 128-weight half of the super-block
    const float4 da0 = *reinterpret_cast<const float4*>(&sS[g][8 * hb]), da1 = *reinterpret_cast<const float4*>(&sS[g][8 * hb + 4]);
    const float4 db0 = *reinterpret_cast<const float4*>(&sS[g + 8][8 * hb]), db1 = *reinterpret_cast<const float4*>(&sS[g + 8][8 * hb + 4]);
    const float ds_a[8] = {da0.x, da0.y, da0.z, da0.w, da1.x, da1.y, da1.z, da1.w};
    const float ds_b[8] = {db0.x, db0.y, db0.z, db0.w, db1.x, db1.y, db1.z, db1.w};
#pragma unroll
    for (int u = 0; u < 2; ++u) {                    // which 16 of the 32 positions l
      const int l0 = 16 * u + 4 * t;
      const uint32_t la0 = lds_word<ODD>(b0 + 64 * hb + l0), la1 = lds_word<ODD>(b0 + 64 * hb + 32 + l0);
      const uint32_t ha = lds_word<ODD>(b0 + 128 + 32 * hb + l0);
      const uint32_t lb0 = lds_word<ODD>(b1 + 64 * hb + l0), lb1 = lds_word<ODD>(b1 + 64 * hb + 32 + l0);
      const uint32_t hb_ = lds_word<ODD>(b1 + 128 + 32 * hb + l0);
#pragma unroll
      for (int quad = 0; quad < 4; ++quad) {         // weights 128*hb + 32*quad + l, sub-block 8*hb + 2*quad + u
        const uint32_t lwa = (quad & 1) ? la1 : la0, lwb = (quad & 1) ? lb1 : lb0;
        const uint32_t na = ((quad & 2) ? lwa >> 4 : lwa) & 0x0f0f0f0fu, nb = ((quad & 2) ? lwb >> 4 : lwb) & 0x0f0f0f0fu;
        // the two high bits of quad q sit at bit 2q of the qh byte; they belong at bit 4
        const uint32_t hsa = quad == 0 ? ha << 4 : quad == 1 ? ha << 2 : quad == 2 ? ha : ha >> 2;
        const uint32_t hsb = quad == 0 ? hb_ << 4 : quad == 1 ? hb_ << 2 : quad == 2 ? hb_ : hb_ >> 2;
        const uint32_t qa = na | (hsa & 0x30303030u), qb = nb | (hsb & 0x30303030u);
        const uint32_t a[4] = {q6_center<T>(__byte_perm(qa, MT::kMagicBytes, 0x4140)), q6_center<T>(__byte_perm(qb, MT::kMagicBytes, 0x4140)),
                               q6_center<T>(__byte_perm(qa, MT::kMagicBytes, 0x4342)), q6_center<T>(__byte_perm(qb, MT::kMagicBytes, 0x4342))};
        const float dsr0 = ds_a[2 * quad + u], dsr1 = ds_b[2 * quad + u];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          // rows >= m read a clamped (valid) row; their accumulator columns are never stored
          const uint2 xb = __ldg(reinterpret_cast<const uint2*>(xrow[nt] + sb * 256 + 128 * hb + 32 * quad + 16 * u));
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
          MT::mma(acc, a, xb.x, xb.y);
          res[nt][0] = fmaf(dsr0, acc[0], res[nt][0]);
          res[nt][2] = fmaf(dsr1, acc[2], res[nt][2]);
          if (MC == 2) {
            res[nt][1] = fmaf(dsr0, acc[1], res[nt][1]);
            res[nt][3] = fmaf(dsr1, acc[3], res[nt][3]);
          }
        }
      }
    }
  }
  __syncwarp();                        // sS is rewritten for the next super-block
}

}  // namespace b200gguf
