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
#include "gemv_q6k_common.cuh"

namespace b200gguf {

constexpr int kQ6Rows = 16;
constexpr int kQ6StageSb = 4;                            // super-blocks per stage (one per warp of a group)
constexpr int kQ6StageSrc = kQ6StageSb * 210;            // 840 B of each row per stage
constexpr int kQ6Chunks = 53;                            // 16-byte chunks of the aligned window (840 + up to 8 B lead)
constexpr int kQ6Pitch = 912;                            // pitch % 128 == 16: 4-byte reads of 8 rows x 4 lanes hit 32 banks
constexpr int kQ6StageBytes = kQ6Rows * kQ6Pitch;        // 14592 B per stage slot
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
