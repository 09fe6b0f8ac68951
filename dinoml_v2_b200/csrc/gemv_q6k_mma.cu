// Fused GGUF decode GEMV ("mma" variant) for Q6_K weights, M = 1..16, float16 / bfloat16 activations.
//
// C[M,N] = A[M,K] * dequant(W[N,K])^T (+ bias) with W streamed once from HBM as packed GGUF blocks.
// HBM-bound: the algorithmic traffic is the packed weight bytes (210 B per 256 weights).
//
// Exact arithmetic on tensor cores: a 6-bit quant q is assembled from its ql nibble and qh bit pair with 32-bit
// logic, turned into a 16-bit float by a byte permute (bf16 0x43qq == 128 + q, fp16 0x64qq == 1024 + q), and the
// offset (MAGIC + 32) is subtracted with one packed subtract, which is exact: the MMA operand is the integer
// q - 32.  A Q6_K scale covers 16 weights = the K extent of one mma.sync.m16n8k16, so each MMA is a whole
// sub-block and its fp32 result is scaled by d * sc[j] afterwards:
//     y[n,m] = sum_j (d[n] * sc[n,j]) * sum_{k in j} (q[n,k] - 32) * x[m,k]
//
// Data movement follows the Q4_K kernel: a CTA owns 16 consecutive weight rows, stages their packed bytes
// HBM -> shared memory with 16-byte cp.async copies in K-stages of 4 super-blocks (one per warp of a warp
// group), several stages in flight, launched with programmatic stream serialization (weights are prefetched
// before the wait on the preceding kernel).  210-byte blocks are only 2-byte aligned: a stage copies the
// 16-byte aligned window around its 840 bytes, and a warp whose block starts 2 bytes off a word boundary
// (every odd block of a row) rebuilds each 32-bit word from two aligned loads with a byte permute.  When rows are
// 16-byte multiples (K % 2048 == 0) the window offset is the same for every row and the phase of a block is known per
// warp; any other K % 256 == 0 runs the RAGGED instantiation, where every row has its own window offset and every
// word load decides its phase at run time.
// Lane (g = lane/4, t = lane%4) feeds rows g and g+8 and, in every 16-wide sub-block, the weights 4t..4t+3.
//
// Behavioural ancestor in the reference: the small-M "wave" kernels of the fused prototype
// (kernels/rocm/src/ck_gguf_q8_gemm.hip:1009-1166); block layout per kernels/cuda/vendor/gguf-cuda
// dequantize.cuh (ql low nibbles / high nibbles, qh bit pairs, 16 int8 scales, fp16 d).
#include "gemv_mma_common.cuh"

namespace b200gguf {

constexpr int kQ6Rows = 16;
constexpr int kQ6StageSb = 4;                            // super-blocks per stage (one per warp of a group)
constexpr int kQ6StageSrc = kQ6StageSb * 210;            // 840 B of each row per stage
constexpr int kQ6Chunks = 53;                            // 16-byte chunks of the aligned window (840 + up to 8 B lead)
constexpr int kQ6Pitch = 912;                            // pitch % 128 == 16: 4-byte reads of 8 rows x 4 lanes hit 32 banks
constexpr int kQ6StageBytes = kQ6Rows * kQ6Pitch;        // 14592 B per stage slot
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

// MXC: activation rows covered (power of two >= m).  NW: warps per CTA (4 or 8); each group of 4 warps walks its own
// sequence of K-stages.  NSTAGE: shared-memory stage slots (dynamic shared memory).
// SLICED: grid.y K slices per row tile, reduced through the cluster's distributed shared memory (see gemv_mma_common.cuh).
// SCATTER: the result also goes to the extra destinations in `peers` (see PeerOut).
// RAGGED: K is any multiple of 256 - weight rows need not be 16-byte multiples (every row then sits at its own phase
// inside its staged window) and the last stage may hold fewer than 4 super-blocks.
template <typename T, int MXC, int NW, int NSTAGE, bool SLICED, bool SCATTER, bool RAGGED>
__global__ void __launch_bounds__(NW * 32)
gemv_q6k_mma_kernel(const T* __restrict__ x, const uint8_t* __restrict__ w, const T* __restrict__ bias, T* __restrict__ y, int m,
                    int n, int k, const PeerOut peers) {
  using MT = MmaType<T>;
  constexpr int NT = MXC > 8 ? 2 : 1;        // n8 tiles of activation rows
  constexpr int MC = MXC == 1 ? 1 : 2;       // accumulator columns a lane keeps per tile
  constexpr int kCols = NT * 8;
  constexpr int SPI = NW / 4;                // stages per iteration (one per warp group)
  constexpr int D = NSTAGE / SPI;            // stage slots per warp group
  static_assert(NSTAGE % SPI == 0 && D >= 2, "each warp group needs at least two stage slots");
  extern __shared__ __align__(16) uint8_t smem_dyn[];
  uint8_t* sW = smem_dyn;                                               // staged packed weights, NSTAGE x kQ6StageBytes
  __shared__ __align__(16) float sS[NW][kQ6Rows][kQ6ScalePitch];        // d * sc per row, sub-block
  // the cross-warp reduction buffer reuses the stage slots once every warp is done with them
  float (*sRed)[kQ6Rows][kCols] = reinterpret_cast<float (*)[kQ6Rows][kCols]>(smem_dyn);
  static_assert(NW * kQ6Rows * kCols * sizeof(float) <= size_t(NSTAGE) * kQ6StageBytes, "reduction buffer must fit");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = warp >> 2, wq = warp & 3, gtid = tid & 127;   // warp group, warp within it, thread within it
  const int g = lane >> 2, t = lane & 3;
  const int r_base = blockIdx.x * kQ6Rows;
  const int nsb = k >> 8;
  const int nstages_all = (nsb + kQ6StageSb - 1) / kQ6StageSb;
  // K slice of this CTA (grid.y = cluster size = slices per row tile)
  const int ks = SLICED ? int(gridDim.y) : 1, kr = SLICED ? int(cluster_rank()) : 0;
  const int per_slice = (nstages_all + ks - 1) / ks;
  const int s_first = kr * per_slice;
  const int nstages = max(0, min(nstages_all, s_first + per_slice) - s_first);
  const int niter = (nstages + SPI - 1) / SPI;
  const int row_bytes = nsb * 210;
  const uint32_t sW_u32 = uint32_t(__cvta_generic_to_shared(sW));

  // Copy assignment inside a warp group: 8 threads per weight row, thread (gtid%8) moves 16-byte chunks
  // (gtid%8) + 8j of the row's window.
  const int cp_row = gtid >> 3, cp_c0 = gtid & 7;
  const int64_t cp_row_off = int64_t(min(r_base + cp_row, n - 1)) * row_bytes;   // byte offset of the copied row in w
  const uint8_t* cp_src = w + cp_row_off;
  const uint32_t cp_dst = sW_u32 + cp_row * kQ6Pitch + cp_c0 * 16;
  const int64_t total_bytes = int64_t(n) * row_bytes;
  auto issue_stage = [&](int ls) {                                     // ls: stage index inside this CTA's slice
    if (ls < nstages) {
      const int s = s_first + ls;
      const uint32_t dst = cp_dst + (ls % NSTAGE) * kQ6StageBytes;
      if (!RAGGED) {
        const int start = (s * kQ6StageSrc) & ~15;                     // window start inside the row
        const uint8_t* src = cp_src + start + cp_c0 * 16;
#pragma unroll
        for (int j = 0; j < 7; ++j) {
          const int c = cp_c0 + 8 * j;
          if (c < kQ6Chunks && start + 16 * c < row_bytes) cp_async16(dst + 128 * j, src + 128 * j);
        }
      } else {
        // window = the 16-byte aligned span of the weight buffer around this row's 840 bytes (w itself is 16-byte
        // aligned); it may run into the next row, never past the end of the buffer
        const int64_t start = (cp_row_off + int64_t(s) * kQ6StageSrc) & ~int64_t(15);
        const uint8_t* src = w + start + cp_c0 * 16;
#pragma unroll
        for (int j = 0; j < 7; ++j) {
          const int c = cp_c0 + 8 * j;
          const int64_t left = total_bytes - (start + 16 * c);
          if (c < kQ6Chunks + 1 && left > 0) {
            if (left >= 16) cp_async16(dst + 128 * j, src + 128 * j);
            else cp_async16_partial(dst + 128 * j, src + 128 * j, int(left));
          }
        }
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int d = 0; d < D; ++d) issue_stage(d * SPI + grp);
  // Weights are constants: they were safe to prefetch.  Everything below reads activations / writes outputs that a
  // preceding kernel in the stream may still be producing / consuming.
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");

  float res[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) res[nt][i] = 0.f;
  const T* xrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) xrow[nt] = x + int64_t(min(nt * 8 + g, m - 1)) * k + 4 * t;

  for (int it = 0; it < niter; ++it) {
    cp_async_wait<D - 2>();
    __syncthreads();                       // this iteration's stages landed; the previous ones are fully consumed
    if (it > 0) issue_stage((it - 1 + D) * SPI + grp); else cp_async_commit();
    const int ls = it * SPI + grp;
    if (ls < nstages) {
      const int s = s_first + ls;
      const uint8_t* slot = sW + (ls % NSTAGE) * kQ6StageBytes;
      const int sb = s * kQ6StageSb + wq;
      if (RAGGED) {
        if (sb < nsb) {
          // row r's window starts (row offset + s * 840) % 16 bytes before its first block of the stage
          auto block_of = [&](int r) {
            const int64_t off = int64_t(min(r_base + r, n - 1)) * row_bytes + int64_t(s) * kQ6StageSrc;
            return slot + r * kQ6Pitch + int(off & 15) + wq * 210;
          };
          q6k_superblock<T, NT, MC, Q6_RUNTIME>(block_of(lane >> 1), block_of(g), block_of(g + 8), sS[warp], xrow, sb, lane, res);
        }
      } else {
        // the stage window starts (s * 840) % 16 bytes before the stage's first block; block wq follows 210 * wq later
        const uint8_t* st = slot + ((s * kQ6StageSrc) & 15) + wq * 210;
        if (wq & 1) q6k_superblock<T, NT, MC, Q6_ODD>(st + (lane >> 1) * kQ6Pitch, st + g * kQ6Pitch, st + (g + 8) * kQ6Pitch, sS[warp], xrow, sb, lane, res);
        else q6k_superblock<T, NT, MC, Q6_ALIGNED>(st + (lane >> 1) * kQ6Pitch, st + g * kQ6Pitch, st + (g + 8) * kQ6Pitch, sS[warp], xrow, sb, lane, res);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();                         // every warp is done with the stage slots: reuse them for the reduction

#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    sRed[warp][g][nt * 8 + 2 * t] = res[nt][0];
    sRed[warp][g][nt * 8 + 2 * t + 1] = res[nt][1];
    sRed[warp][g + 8][nt * 8 + 2 * t] = res[nt][2];
    sRed[warp][g + 8][nt * 8 + 2 * t + 1] = res[nt][3];
  }
  __syncthreads();
  __shared__ float sOut[kQ6Rows * MXC];    // this CTA's sums; read by the rank-0 CTA of the cluster when K is sliced
  for (int idx = tid; idx < kQ6Rows * MXC; idx += NW * 32) {
    const int r = idx & (kQ6Rows - 1), c = idx >> 4;
    float v = 0.f;
#pragma unroll
    for (int wv = 0; wv < NW; ++wv) v += sRed[wv][r][c];
    sOut[idx] = v;
  }
  if (SLICED) cluster_barrier(); else __syncthreads();
  if (kr == 0) {
    for (int idx = tid; idx < kQ6Rows * MXC; idx += NW * 32) {
      const int r = idx & (kQ6Rows - 1), c = idx >> 4;
      const int row = r_base + r;
      if (row >= n || c >= m) continue;
      float v = sOut[idx];
      if (SLICED)
        for (int peer = 1; peer < ks; ++peer) v += ld_cluster_f32(&sOut[idx], uint32_t(peer));
      int64_t at = int64_t(c) * n + row;
      if (peers.act != ACT_NONE) {
        // gated pair: rows r < 8 of the tile belong to the first matrix, r + 8 to the second; output has n / 2 columns
        if (r >= 8) continue;
        float u = sOut[idx + 8];
        if (SLICED)
          for (int peer = 1; peer < ks; ++peer) u += ld_cluster_f32(&sOut[idx + 8], uint32_t(peer));
        v = gate_activation(v, peers.act) * u;
        at = int64_t(c) * (n >> 1) + (blockIdx.x * 8 + r);
      } else if (bias != nullptr) {
        v += MT::to_float(bias[row]);
      }
      const T out = MT::from_float(v);
      y[at] = out;
      if (SCATTER) {
#pragma unroll
        for (int pi = 0; pi < 8; ++pi)
          if (pi < peers.count) static_cast<T*>(peers.ptr[pi])[at] = out;
      }
    }
  }
  if (SLICED) cluster_barrier();           // peers keep their shared memory alive until rank 0 has read it
}

template <typename T, int MXC, int NW, int NSTAGE, bool SLICED>
static int launch_q6k_cfg(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, const PeerOut& peers, cudaStream_t s) {
  const int tiles = (n + kQ6Rows - 1) / kQ6Rows;
  constexpr size_t smem = size_t(NSTAGE) * kQ6StageBytes;
  const bool ragged = k % 2048 != 0;          // rows that are not 16-byte multiples, or a last stage of fewer than 4 super-blocks
  auto kern = ragged ? (peers.count > 0 ? gemv_q6k_mma_kernel<T, MXC, NW, NSTAGE, SLICED, true, true> : gemv_q6k_mma_kernel<T, MXC, NW, NSTAGE, SLICED, false, true>)
                     : (peers.count > 0 ? gemv_q6k_mma_kernel<T, MXC, NW, NSTAGE, SLICED, true, false> : gemv_q6k_mma_kernel<T, MXC, NW, NSTAGE, SLICED, false, false>);
  static SmemOptIn granted[4];          // per kernel (plain / scatter, aligned / ragged), per device
  if (!smem_opt_in(kern, smem, granted[(peers.count > 0 ? 1 : 0) + (ragged ? 2 : 0)])) return RC_LAUNCH;
  const int ks = SLICED ? gemv_k_slices(tiles, ((k >> 8) + kQ6StageSb - 1) / kQ6StageSb, NSTAGE) : 1;
  const cudaError_t err = gemv_launch(kern, tiles, ks, NW * 32, smem, s, static_cast<const T*>(a), static_cast<const uint8_t*>(b),
                                      static_cast<const T*>(bias), static_cast<T*>(c), m, n, k, peers);
  return err == cudaSuccess ? RC_OK : RC_LAUNCH;
}

template <typename T, int MXC>
static int launch_q6k_m(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, const PeerOut& peers, cudaStream_t s) {
  if constexpr (MXC <= 8) {
    // Few row tiles (all CTAs resident at two per SM): six stage slots per CTA keep more bytes in flight.  Many row
    // tiles: four slots, so that three CTAs fit on an SM.
    int sm_count = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if ((n + kQ6Rows - 1) / kQ6Rows <= 2 * sm_count) return launch_q6k_cfg<T, MXC, 8, 6, false>(a, b, bias, c, m, n, k, peers, s);
    return launch_q6k_cfg<T, MXC, 8, 4, false>(a, b, bias, c, m, n, k, peers, s);
  }
  return launch_q6k_cfg<T, MXC, 4, 3, true>(a, b, bias, c, m, n, k, peers, s);
}

template <typename T>
static int launch_q6k(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, const PeerOut& peers, cudaStream_t s) {
  if (m == 1) return launch_q6k_m<T, 1>(a, b, bias, c, m, n, k, peers, s);
  if (m == 2) return launch_q6k_m<T, 2>(a, b, bias, c, m, n, k, peers, s);
  if (m <= 4) return launch_q6k_m<T, 4>(a, b, bias, c, m, n, k, peers, s);
  if (m <= 8) return launch_q6k_m<T, 8>(a, b, bias, c, m, n, k, peers, s);
  return launch_q6k_m<T, 16>(a, b, bias, c, m, n, k, peers, s);
}

bool gemv_q6k_mma_supports(int dtype, int m, int k) {
  return (dtype == DINO_BF16 || dtype == DINO_F16) && m >= 1 && m <= 16 && k % 256 == 0;
}

int gemv_q6k_mma(const void* a, const void* b, const void* bias, void* c, int dtype, int m, int n, int k, const PeerOut& peers, cudaStream_t s) {
  return dtype == DINO_BF16 ? launch_q6k<__nv_bfloat16>(a, b, bias, c, m, n, k, peers, s) : launch_q6k<__half>(a, b, bias, c, m, n, k, peers, s);
}

}  // namespace b200gguf
