// Fused GGUF decode GEMV ("mma" variant), M = 1..16, float16 / bfloat16 activations, Q4_K weights (the Q6_K kernel
// is in gemv_q6k_mma.cu; the variant's dispatch is at the end of this file).
//
// C[M,N] = A[M,K] * dequant(W[N,K])^T (+ bias) with W streamed once from HBM as packed GGUF blocks.
// HBM-bound: the algorithmic traffic is the packed weight bytes (144 B per 256 weights).
//
// How the arithmetic stays exact while running on tensor cores: the 4-bit quants are turned into
// 16-bit floats with a bit trick (bf16 0x4300|q == 128+q; fp16 0x6400|q == 1024+q, minus 1024),
// multiplied against the unmodified 16-bit activations by mma.sync.m16n8k16 with fp32 accumulation,
// and only then scaled in fp32 per 32-wide sub-block j:
//     y[n,m] = sum_j ds[n,j] * S'[n,m,j]  -  sum_j (MAGIC*ds[n,j] + dm[n,j]) * X[m,j]
// with S' = sum_k x*(MAGIC+q) from the MMA, X[m,j] the sum of the sub-block's activations (computed
// once per CTA into shared memory), ds = d*sc and dm = dmin*min the sub-block scale and min.
//
// Data movement: a CTA of 4 warps owns 16 consecutive weight rows (one MMA M-tile).  Their packed
// bytes are staged HBM -> shared memory with 16-byte cp.async copies in K-stages of 4 super-blocks
// (16 rows x 576 B), four stages in flight per CTA (the whole row set for K = 4096), so every SM keeps
// >150 KB of reads outstanding without holding them in registers.  The kernel is launched with programmatic
// stream serialization: it prefetches its (constant) weights first and only then waits for the preceding
// kernel in the stream (`griddepcontrol.wait`) before touching activations or outputs, so consecutive
// quantized linears overlap one launch's ramp-up with the previous one's tail.  Within a stage warp w unpacks super-block w.  Lane
// (g = lane/4, t = lane%4) feeds rows g and g+8: per 64-weight group it reads the 8 quant bytes
// [8t, 8t+8) of each row, which puts all 16 K-slots of every MMA inside one sub-block.  The row pitch
// in shared memory (608 B) makes those 8-byte reads bank-conflict free.  The 16 header bytes of each
// (row, super-block) are decoded by a lane pair (lane/2 = row, lane%2 = which 4 sub-blocks) into ds,
// shared through shared memory, while the same lane folds the min / MAGIC term against X directly.
// The four warps' partial rows are summed through shared memory at the end.
//
// Behavioural ancestor in the reference: the small-M "wave" kernels of the fused prototype
// (kernels/rocm/src/ck_gguf_q8_gemm.hip:1009-1166); the reference's CUDA path instead dequantizes the
// whole weight and runs a dense Sm80 GEMM (src/dinoml/lowering/ops/gemm.py:729-749).
#include "gemv_mma_common.cuh"

namespace b200gguf {

int check_gemm_args(const void* a, const void* b, const void* c, int qtype, int dtype, int m, int n, int k);
bool gemv_q6k_mma_supports(int dtype, int m, int k);
bool gemv_q8_0_mma_supports(int dtype, int m, int k);
int gemv_q8_0_mma(const void* a, const void* b, const void* bias, void* c, int dtype, int m, int n, int k, cudaStream_t s);
int gemv_q6k_mma(const void* a, const void* b, const void* bias, void* c, int dtype, int m, int n, int k, const PeerOut& peers, cudaStream_t s);

constexpr int kGemvWarps = 4;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kGemvRows = 16;
constexpr int kStageSb = 4;                              // super-blocks per stage (one per warp)
constexpr int kRowChunks = kStageSb * 9;                 // 16-byte chunks per row per stage (4 x 144 B)
constexpr int kRowPitch = kStageSb * 144 + 32;           // 608 B: 8-byte reads of 8 rows x 4 lanes hit 32 banks
constexpr int kStageBytes = kGemvRows * kRowPitch;       // 9728 B per stage slot

// MXC: activation rows covered (power of two >= m).  NW: warps per CTA (4 or 8); each group of 4 warps walks its own
// sequence of K-stages (group p takes stages p, p + NW/4, ...), so an 8-warp CTA unpacks two stages at a time.
// NSTAGE: shared-memory stage slots.  Dynamic shared memory: weight stages, then X[MXC][k/32] floats.
// SLICED: grid.y K slices per row tile, reduced through the cluster's distributed shared memory (see gemv_mma_common.cuh).
// SCATTER: the result also goes to the extra destinations in `peers` (see PeerOut).
template <typename T, int MXC, int NW, int NSTAGE, bool SLICED, bool SCATTER>
__global__ void __launch_bounds__(NW * 32)
gemv_q4k_mma_kernel(const T* __restrict__ x, const uint8_t* __restrict__ w, const T* __restrict__ bias,
                    T* __restrict__ y, int m, int n, int k, const PeerOut peers) {
  using MT = MmaType<T>;
  constexpr int NT = MXC > 8 ? 2 : 1;        // n8 tiles of activation rows
  constexpr int MC = MXC == 1 ? 1 : 2;       // accumulator columns a lane keeps per tile
  constexpr int kCols = NT * 8;
  constexpr int SPI = NW / 4;                // stages per iteration (one per warp group)
  constexpr int D = NSTAGE / SPI;            // stage slots per warp group
  static_assert(NSTAGE % SPI == 0 && D >= 2, "each warp group needs at least two stage slots");
  extern __shared__ __align__(16) uint8_t smem_dyn[];
  uint8_t* sW = smem_dyn;                                                 // staged packed weights, NSTAGE x kStageBytes
  float* sX = reinterpret_cast<float*>(smem_dyn + NSTAGE * kStageBytes);  // [MXC][k/32]
  __shared__ __align__(16) float sS[NW][kGemvRows][8];                    // ds per row, sub-block
  // From four activation rows on, the per-sub-block activation sums come from the tensor cores (one more MMA pair per
  // sub-block: the activation fragment against an all-ones operand) instead of a table every CTA builds from M * K
  // activations before its first stage; the folded offsets (MAGIC * ds + dmin * min) then wait in sK.
  constexpr bool kOnes = MXC >= 4;
  __shared__ __align__(16) float sK[kOnes ? NW : 1][kOnes ? kGemvRows : 1][8];
  // the cross-warp reduction buffers reuse the stage slots once every warp is done with them
  float (*sRed)[kGemvRows][kCols] = reinterpret_cast<float (*)[kGemvRows][kCols]>(smem_dyn);
  float (*sXt)[kGemvRows][2][MXC] = reinterpret_cast<float (*)[kGemvRows][2][MXC]>(smem_dyn + NW * kGemvRows * kCols * sizeof(float));
  static_assert(NW * kGemvRows * (kCols + 2 * MXC) * sizeof(float) <= size_t(NSTAGE) * kStageBytes, "reduction buffers must fit");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = warp >> 2, wq = warp & 3, gtid = tid & 127;   // warp group, warp within it, thread within it
  const int g = lane >> 2, t = lane & 3;
  const int r_base = blockIdx.x * kGemvRows;
  const int nsb = k >> 8, nsub = k >> 5;
  const int nstages_all = (nsb + kStageSb - 1) / kStageSb;
  // K slice of this CTA (grid.y = cluster size = slices per row tile)
  const int ks = SLICED ? int(gridDim.y) : 1, kr = SLICED ? int(cluster_rank()) : 0;
  const int per_slice = (nstages_all + ks - 1) / ks;
  const int s_first = kr * per_slice;
  const int nstages = max(0, min(nstages_all, s_first + per_slice) - s_first);
  const int niter = (nstages + SPI - 1) / SPI;
  const int64_t row_bytes = int64_t(nsb) * 144;
  const uint32_t sW_u32 = uint32_t(__cvta_generic_to_shared(sW));

  // Copy assignment inside a warp group: 8 threads per weight row, thread (gtid%8) moves 16-byte chunks
  // (gtid%8) + 8j of the row's 36 chunks per stage.
  const int cp_row = gtid >> 3, cp_c0 = gtid & 7;
  const uint8_t* cp_src = w + int64_t(min(r_base + cp_row, n - 1)) * row_bytes + cp_c0 * 16;
  const uint32_t cp_dst = sW_u32 + cp_row * kRowPitch + cp_c0 * 16;
  auto issue_stage = [&](int ls) {                                     // ls: stage index inside this CTA's slice
    if (ls < nstages) {
      const int s = s_first + ls;
      const int valid_chunks = min(kStageSb, nsb - s * kStageSb) * 9;
      const uint8_t* src = cp_src + int64_t(s) * (kStageSb * 144);
      const uint32_t dst = cp_dst + (ls % NSTAGE) * kStageBytes;
#pragma unroll
      for (int j = 0; j < 5; ++j)
        if (cp_c0 + 8 * j < valid_chunks) cp_async16(dst + 128 * j, src + 128 * j);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int d = 0; d < D; ++d) issue_stage(d * SPI + grp);
  // Weights are constants: they were safe to prefetch.  Everything below reads activations / writes outputs that a
  // preceding kernel in the stream may still be producing / consuming.
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");

  // X[c][j] = sum of activations of row c over sub-block j (rows >= m are zero), for the sub-blocks of this K slice.
  const int j_first = s_first * (kStageSb * 8), j_count = min(nsub - j_first, nstages * (kStageSb * 8));
  for (int i = tid; !kOnes && i < j_count * MXC; i += NW * 32) {
    const int c = i / j_count, j = j_first + (i - c * j_count);
    const int idx = c * nsub + j;
    float s = 0.f;
    if (c < m) {
      const uint4* px = reinterpret_cast<const uint4*>(x + int64_t(c) * k + int64_t(j) * 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) s += MT::sum8(__ldg(px + i));
    }
    sX[idx] = s;
  }

  float res[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) res[nt][i] = 0.f;
  float xt[MXC];
#pragma unroll
  for (int c = 0; c < MXC; ++c) xt[c] = 0.f;

  const int srow = lane >> 1, shalf = lane & 1;   // scale-decode role of this lane
  const T* xrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) xrow[nt] = x + int64_t(min(nt * 8 + g, m - 1)) * k + 8 * t;

  for (int it = 0; it < niter; ++it) {
    cp_async_wait<D - 2>();
    __syncthreads();                       // this iteration's stages landed; the previous ones are fully consumed
    if (it > 0) issue_stage((it - 1 + D) * SPI + grp); else cp_async_commit();
    const int ls = it * SPI + grp;
    const int sb = (s_first + ls) * kStageSb + wq;
    if (ls < nstages && sb < nsb) {
      const uint8_t* st = sW + (ls % NSTAGE) * kStageBytes + wq * 144;
      {  // lane pair (srow, shalf): 4 sub-block scales -> ds to shared memory, min/MAGIC term folded against X
        const uint4 hdr = *reinterpret_cast<const uint4*>(st + srow * kRowPitch);
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
        *reinterpret_cast<float4*>(&sS[warp][srow][4 * shalf]) = dsv;
        if constexpr (kOnes) {
          *reinterpret_cast<float4*>(&sK[warp][srow][4 * shalf]) = make_float4(kk[0], kk[1], kk[2], kk[3]);
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
      const float4 dsa0 = *reinterpret_cast<const float4*>(&sS[warp][g][0]);
      const float4 dsa1 = *reinterpret_cast<const float4*>(&sS[warp][g][4]);
      const float4 dsb0 = *reinterpret_cast<const float4*>(&sS[warp][g + 8][0]);
      const float4 dsb1 = *reinterpret_cast<const float4*>(&sS[warp][g + 8][4]);
      const float ds_a[8] = {dsa0.x, dsa0.y, dsa0.z, dsa0.w, dsa1.x, dsa1.y, dsa1.z, dsa1.w};
      const float ds_b[8] = {dsb0.x, dsb0.y, dsb0.z, dsb0.w, dsb1.x, dsb1.y, dsb1.z, dsb1.w};
      const uint8_t* q0p = st + g * kRowPitch + 16 + 8 * t;
      const uint8_t* q1p = q0p + 8 * kRowPitch;
#pragma unroll
      for (int G = 0; G < 4; ++G) {
        const uint2 q0 = *reinterpret_cast<const uint2*>(q0p + 32 * G);
        const uint2 q1 = *reinterpret_cast<const uint2*>(q1p + 32 * G);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t n0x = (h ? q0.x >> 4 : q0.x) & 0x0f0f0f0fu, n0y = (h ? q0.y >> 4 : q0.y) & 0x0f0f0f0fu;
          const uint32_t n1x = (h ? q1.x >> 4 : q1.x) & 0x0f0f0f0fu, n1y = (h ? q1.y >> 4 : q1.y) & 0x0f0f0f0fu;
          const uint32_t a_lo[4] = {MT::fix(__byte_perm(n0x, MT::kMagicBytes, 0x4140)), MT::fix(__byte_perm(n1x, MT::kMagicBytes, 0x4140)),
                                    MT::fix(__byte_perm(n0x, MT::kMagicBytes, 0x4342)), MT::fix(__byte_perm(n1x, MT::kMagicBytes, 0x4342))};
          const uint32_t a_hi[4] = {MT::fix(__byte_perm(n0y, MT::kMagicBytes, 0x4140)), MT::fix(__byte_perm(n1y, MT::kMagicBytes, 0x4140)),
                                    MT::fix(__byte_perm(n0y, MT::kMagicBytes, 0x4342)), MT::fix(__byte_perm(n1y, MT::kMagicBytes, 0x4342))};
          const float dsr0 = ds_a[2 * G + h], dsr1 = ds_b[2 * G + h];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            // rows >= m read a clamped (valid) row; their accumulator columns are never stored
            const uint4 xb = __ldg(reinterpret_cast<const uint4*>(xrow[nt] + sb * 256 + 64 * G + 32 * h));
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            MT::mma(acc, a_lo, xb.x, xb.y);
            MT::mma(acc, a_hi, xb.z, xb.w);
            res[nt][0] = fmaf(dsr0, acc[0], res[nt][0]);
            res[nt][2] = fmaf(dsr1, acc[2], res[nt][2]);
            if (MC == 2) {
              res[nt][1] = fmaf(dsr0, acc[1], res[nt][1]);
              res[nt][3] = fmaf(dsr1, acc[3], res[nt][3]);
            }
            if constexpr (kOnes) {
              const uint32_t ones[4] = {MT::kOnePair, MT::kOnePair, MT::kOnePair, MT::kOnePair};
              float sx[4] = {0.f, 0.f, 0.f, 0.f};
              MT::mma(sx, ones, xb.x, xb.y);
              MT::mma(sx, ones, xb.z, xb.w);
              const float kk0 = sK[warp][g][2 * G + h], kk1 = sK[warp][g + 8][2 * G + h];
              res[nt][0] = fmaf(-kk0, sx[0], res[nt][0]);
              res[nt][2] = fmaf(-kk1, sx[0], res[nt][2]);
              if (MC == 2) {
                res[nt][1] = fmaf(-kk0, sx[1], res[nt][1]);
                res[nt][3] = fmaf(-kk1, sx[1], res[nt][3]);
              }
            }
          }
        }
      }
      __syncwarp();                        // sS (and sK) are rewritten in the next iteration
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
#pragma unroll
  for (int c = 0; c < MXC; ++c) sXt[warp][srow][shalf][c] = xt[c];
  __syncthreads();
  __shared__ float sOut[kGemvRows * MXC];  // this CTA's sums; read by the rank-0 CTA of the cluster when K is sliced
  for (int idx = tid; idx < kGemvRows * MXC; idx += NW * 32) {
    const int r = idx & (kGemvRows - 1), c = idx >> 4;
    float v = 0.f, xs = 0.f;
#pragma unroll
    for (int wv = 0; wv < NW; ++wv) {
      v += sRed[wv][r][c];
      xs += sXt[wv][r][0][c] + sXt[wv][r][1][c];
    }
    sOut[idx] = v - xs;
  }
  if (SLICED) cluster_barrier(); else __syncthreads();
  if (kr == 0) {
    for (int idx = tid; idx < kGemvRows * MXC; idx += NW * 32) {
      const int r = idx & (kGemvRows - 1), c = idx >> 4;
      const int row = r_base + r;
      if (row >= n || c >= m) continue;
      float v = sOut[idx];
      if (SLICED)
        for (int peer = 1; peer < ks; ++peer) v += ld_cluster_f32(&sOut[idx], uint32_t(peer));
      int64_t at = int64_t(c) * n + row;
      if (bias != nullptr) v += MT::to_float(bias[row]);
      if (peers.act != ACT_NONE) {
        // gated pair: rows r < 8 of the tile belong to the first matrix, r + 8 to the second; output has n / 2 columns
        if (r >= 8) continue;
        float u = sOut[idx + 8];
        if (SLICED)
          for (int peer = 1; peer < ks; ++peer) u += ld_cluster_f32(&sOut[idx + 8], uint32_t(peer));
        // bias interleaved like the rows: bias0 of the gate row (added above), bias1 of its up row
        if (bias != nullptr) u += MT::to_float(bias[row + 8]);
        v = gate_activation(v, peers.act) * u;
        at = int64_t(c) * (n >> 1) + (blockIdx.x * 8 + r);
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
static int launch_q4k_cfg(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, const PeerOut& peers, cudaStream_t s) {
  const int tiles = (n + kGemvRows - 1) / kGemvRows;
  const size_t smem = size_t(NSTAGE) * kStageBytes + (MXC >= 4 ? 0 : size_t(k / 32) * MXC * sizeof(float));   // the sum table of M <= 2
  if (smem > 200 * 1024) return RC_RANGE;
  auto kern = peers.count > 0 ? gemv_q4k_mma_kernel<T, MXC, NW, NSTAGE, SLICED, true> : gemv_q4k_mma_kernel<T, MXC, NW, NSTAGE, SLICED, false>;
  static SmemOptIn granted[2];          // per kernel (plain / scatter), per device
  if (!smem_opt_in(kern, smem, granted[peers.count > 0 ? 1 : 0])) return RC_LAUNCH;
  const int ks = SLICED ? gemv_k_slices(tiles, ((k >> 8) + kStageSb - 1) / kStageSb, NSTAGE) : 1;
  const cudaError_t err = gemv_launch(kern, tiles, ks, NW * 32, smem, s, static_cast<const T*>(a), static_cast<const uint8_t*>(b),
                                      static_cast<const T*>(bias), static_cast<T*>(c), m, n, k, peers);
  return err == cudaSuccess ? RC_OK : RC_LAUNCH;
}

// M <= 2: 8 warps and 4 stage slots, one CTA per row tile over the whole K (78 registers: 3 CTAs per SM).  M = 3..8:
// the same CTA shape with K sliced across a cluster, so that a CTA's whole slice is in flight from its first
// instruction on (measured 12.8 vs 14.8 us at M = 4 on [11008 x 4096]).  M = 9..16 needs more shared memory for X and
// the reduction: 4 warps, 3 slots, sliced.
template <typename T, int MXC>
static int launch_q4k_m(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, const PeerOut& peers, cudaStream_t s) {
  if (MXC <= 2 && k >= 2048) return launch_q4k_cfg<T, MXC, 8, 4, false>(a, b, bias, c, m, n, k, peers, s);
  if (MXC <= 2) return launch_q4k_cfg<T, MXC, 4, 4, false>(a, b, bias, c, m, n, k, peers, s);
  if (MXC <= 8) return launch_q4k_cfg<T, MXC, 8, 4, true>(a, b, bias, c, m, n, k, peers, s);
  return launch_q4k_cfg<T, MXC, 4, 3, true>(a, b, bias, c, m, n, k, peers, s);
}

template <typename T>
static int launch_q4k(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, const PeerOut& peers, cudaStream_t s) {
  if (m == 1) return launch_q4k_m<T, 1>(a, b, bias, c, m, n, k, peers, s);
  if (m == 2) return launch_q4k_m<T, 2>(a, b, bias, c, m, n, k, peers, s);
  if (m <= 4) return launch_q4k_m<T, 4>(a, b, bias, c, m, n, k, peers, s);
  if (m <= 8) return launch_q4k_m<T, 8>(a, b, bias, c, m, n, k, peers, s);
  return launch_q4k_m<T, 16>(a, b, bias, c, m, n, k, peers, s);
}

// Which (qtype, dtype, m, k) the mma variant covers.
bool gemv_mma_supports(int qtype, int dtype, int m, int n, int k) {
  (void)n;
  if (qtype == QTYPE_Q6_K) return gemv_q6k_mma_supports(dtype, m, k);
  if (qtype == QTYPE_Q8_0) return gemv_q8_0_mma_supports(dtype, m, k);
  return qtype == QTYPE_Q4_K && (dtype == DINO_BF16 || dtype == DINO_F16) && m >= 1 && m <= 16 && k % 256 == 0;
}

// peers: extra destinations of the result (null = none); see PeerOut.
int gemm_rcr_mma_peers(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                       const PeerOut* peer_out, cudaStream_t s) {
  const PeerOut peers = peer_out != nullptr ? *peer_out : no_peers();
  if (int rc = check_gemm_args(a, b, c, qtype, dtype, m, n, k)) return rc;
  if (dtype == DINO_F32) return RC_DTYPE;
  if (m > 16) return RC_RANGE;
  if (qtype != QTYPE_Q4_K && qtype != QTYPE_Q6_K && qtype != QTYPE_Q8_0) return RC_QTYPE;
  if (!gemv_mma_supports(qtype, dtype, m, n, k)) return RC_ALIGN;   // Q8_0 with K % 256 != 0
  if ((reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(a)) & 15) return RC_ALIGN;  // 16-byte cp.async sources, vector loads
  if (qtype == QTYPE_Q6_K) return gemv_q6k_mma(a, b, bias, c, dtype, m, n, k, peers, s);
  if (qtype == QTYPE_Q8_0) {
    if (peers.count > 0 || peers.act != ACT_NONE) return RC_RANGE;   // no scatter / gated epilogue for Q8_0
    return gemv_q8_0_mma(a, b, bias, c, dtype, m, n, k, s);
  }
  return dtype == DINO_BF16 ? launch_q4k<__nv_bfloat16>(a, b, bias, c, m, n, k, peers, s)
                            : launch_q4k<__half>(a, b, bias, c, m, n, k, peers, s);
}

int gemm_rcr_mma(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                 cudaStream_t s) {
  return gemm_rcr_mma_peers(a, b, bias, c, qtype, dtype, m, n, k, nullptr, s);
}

}  // namespace b200gguf
