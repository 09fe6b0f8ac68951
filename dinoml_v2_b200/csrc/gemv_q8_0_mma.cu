// Fused GGUF decode GEMV ("mma" variant) for Q8_0 weights, M = 1..16, float16 / bfloat16 activations.
//
// C[M,N] = A[M,K] * dequant(W[N,K])^T (+ bias) with W streamed once from HBM as packed GGUF blocks.
// HBM-bound: the algorithmic traffic is the packed weight bytes (34 B per 32 weights: fp16 d + 32 int8).
//
// Exact arithmetic on tensor cores: an int8 quant does not fit the byte-permute trick of the K-quant kernels in one
// piece (bf16 0x4300 | v is exact only for v < 128), so it is split into nibbles, q = 16 h + l with l = q & 15 in
// [0, 15] and h = q >> 4 in [-8, 7]; the high nibble of the byte xor 8 is h + 8 in [0, 15].  Both nibbles become
// 16-bit floats MAGIC + l and MAGIC + 8 + h (bf16 MAGIC = 128; fp16 1024, removed exactly before the MMA) and feed
// two mma.sync.m16n8k16 per 16 weights against the unmodified activations, fp32 accumulation; per 32-weight block
//     y[n,m] += d[n] * (16 * S_h + S_l)  -  d[n] * (16 * (MAGIC' + 8) + MAGIC') * X[m]
// with S_* the MMA sums, X[m] the sum of the block's activations (M <= 2: a table computed once per CTA; M >= 4: one more
// MMA of the activation fragment against an all-ones operand) and MAGIC' the part of the magic that is still in the
// operand (128 for bf16, 0 for fp16).
//
// Data movement follows the Q4_K kernel: a CTA owns 16 consecutive weight rows and stages their packed bytes
// HBM -> shared memory with 16-byte cp.async copies in K-stages of 4 x 256 weights (one 272-byte unit of 8 blocks per
// warp of a warp group; rows and units are 16-byte multiples whenever K % 256 == 0), launched with programmatic
// stream serialization.  Inside a unit block i starts at byte 34 i, so its quants are word aligned for odd i and two
// bytes off for even i: those words are rebuilt from two aligned loads with a byte permute.
// Lane (g = lane/4, t = lane%4) feeds rows g and g+8 and, in every 16-weight half of a block, the weights 4t..4t+3.
//
// Behavioural ancestor in the reference: the Q8_0 "wave" kernels of the fused prototype
// (kernels/rocm/src/ck_gguf_q8_gemm.hip:1009-1166, block struct :20-25, value() :728-730).
#include "gemv_mma_common.cuh"

namespace b200gguf {

constexpr int kQ8Rows = 16;
constexpr int kQ8StageUnits = 4;                         // 256-weight units per stage (one per warp of a group)
constexpr int kQ8UnitBytes = 8 * 34;                     // 272 B
constexpr int kQ8StageSrc = kQ8StageUnits * kQ8UnitBytes;   // 1088 B of each row per stage = 68 chunks of 16 B
constexpr int kQ8Pitch = 1168;                           // pitch % 128 == 16: 4-byte reads of 8 rows x 4 lanes hit 32 banks
constexpr int kQ8StageBytes = kQ8Rows * kQ8Pitch;        // 18688 B per stage slot

// 32-bit word at a shared-memory address that is 4-byte aligned (ODD = false) or 2 bytes past alignment.
template <bool ODD>
__device__ __forceinline__ uint32_t q8_word(const uint8_t* p) {
  if (!ODD) return *reinterpret_cast<const uint32_t*>(p);
  const uint32_t* q = reinterpret_cast<const uint32_t*>(p - 2);
  return __byte_perm(q[0], q[1], 0x5432);
}

// One block (32 weights) of rows g and g+8: four MMAs per activation tile, then the fp32 scaling.
// ONES: the block's activation sums come from one more MMA per 16 weights (the activation fragment against an all-ones
// operand) and the offset is folded here; otherwise the caller folds it against a table of sums.
template <typename T, int NT, int MC, bool ODD, bool ONES>
__device__ __forceinline__ void q8_block(const uint8_t* b0, const uint8_t* b1, const T* const (&xp)[NT], int t, float (&res)[NT][4]) {
  using MT = MmaType<T>;
  constexpr float kOffset = 17.f * MT::kMagic + 128.f;   // 16 * (MAGIC' + 8) + MAGIC': what one unit of X is worth
  const uint32_t ones[4] = {MT::kOnePair, MT::kOnePair, MT::kOnePair, MT::kOnePair};
  float sx[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) sx[nt][i] = 0.f;
  const float d0 = half_bits_to_float(*reinterpret_cast<const uint16_t*>(b0));
  const float d1 = half_bits_to_float(*reinterpret_cast<const uint16_t*>(b1));
  float lo[NT][4], hi[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) lo[nt][i] = hi[nt][i] = 0.f;
#pragma unroll
  for (int c = 0; c < 2; ++c) {                      // 16-weight half of the block
    const uint32_t w0 = q8_word<ODD>(b0 + 2 + 16 * c + 4 * t), w1 = q8_word<ODD>(b1 + 2 + 16 * c + 4 * t);
    const uint32_t l0 = w0 & 0x0f0f0f0fu, l1 = w1 & 0x0f0f0f0fu;
    const uint32_t h0 = ((w0 >> 4) & 0x0f0f0f0fu) ^ 0x08080808u, h1 = ((w1 >> 4) & 0x0f0f0f0fu) ^ 0x08080808u;
    const uint32_t a_lo[4] = {MT::fix(__byte_perm(l0, MT::kMagicBytes, 0x4140)), MT::fix(__byte_perm(l1, MT::kMagicBytes, 0x4140)),
                              MT::fix(__byte_perm(l0, MT::kMagicBytes, 0x4342)), MT::fix(__byte_perm(l1, MT::kMagicBytes, 0x4342))};
    const uint32_t a_hi[4] = {MT::fix(__byte_perm(h0, MT::kMagicBytes, 0x4140)), MT::fix(__byte_perm(h1, MT::kMagicBytes, 0x4140)),
                              MT::fix(__byte_perm(h0, MT::kMagicBytes, 0x4342)), MT::fix(__byte_perm(h1, MT::kMagicBytes, 0x4342))};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      // rows >= m read a clamped (valid) row; their accumulator columns are never stored
      const uint2 xb = __ldg(reinterpret_cast<const uint2*>(xp[nt] + 16 * c));
      MT::mma(lo[nt], a_lo, xb.x, xb.y);
      MT::mma(hi[nt], a_hi, xb.x, xb.y);
      if constexpr (ONES) MT::mma(sx[nt], ones, xb.x, xb.y);
    }
  }
  if constexpr (ONES) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      lo[nt][0] = fmaf(-kOffset, sx[nt][0], lo[nt][0]);
      lo[nt][2] = fmaf(-kOffset, sx[nt][0], lo[nt][2]);
      if (MC == 2) {
        lo[nt][1] = fmaf(-kOffset, sx[nt][1], lo[nt][1]);
        lo[nt][3] = fmaf(-kOffset, sx[nt][1], lo[nt][3]);
      }
    }
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    res[nt][0] = fmaf(d0, fmaf(16.f, hi[nt][0], lo[nt][0]), res[nt][0]);
    res[nt][2] = fmaf(d1, fmaf(16.f, hi[nt][2], lo[nt][2]), res[nt][2]);
    if (MC == 2) {
      res[nt][1] = fmaf(d0, fmaf(16.f, hi[nt][1], lo[nt][1]), res[nt][1]);
      res[nt][3] = fmaf(d1, fmaf(16.f, hi[nt][3], lo[nt][3]), res[nt][3]);
    }
  }
}

// MXC: activation rows covered (power of two >= m).  NW: warps per CTA (4 or 8); each group of 4 warps walks its own
// sequence of K-stages.  NSTAGE: shared-memory stage slots.  Dynamic shared memory: weight stages, then X[MXC][k/32].
template <typename T, int MXC, int NW, int NSTAGE>
__global__ void __launch_bounds__(NW * 32)
gemv_q8_0_mma_kernel(const T* __restrict__ x, const uint8_t* __restrict__ w, const T* __restrict__ bias, T* __restrict__ y, int m,
                     int n, int k) {
  using MT = MmaType<T>;
  constexpr int NT = MXC > 8 ? 2 : 1;        // n8 tiles of activation rows
  constexpr int MC = MXC == 1 ? 1 : 2;       // accumulator columns a lane keeps per tile
  constexpr int kCols = NT * 8;
  constexpr int SPI = NW / 4;                // stages per iteration (one per warp group)
  constexpr int D = NSTAGE / SPI;            // stage slots per warp group
  constexpr float kOffset = 17.f * MT::kMagic + 128.f;   // 16 * (MAGIC' + 8) + MAGIC': what one unit of X is worth
  // From four activation rows on the activation sums come from the tensor cores (see q8_block): building the table costs
  // every 16-row CTA M * K activation reads, as many bytes as its weights at M = 8.
  constexpr bool kOnes = MXC >= 4;
  static_assert(NSTAGE % SPI == 0 && D >= 2, "each warp group needs at least two stage slots");
  extern __shared__ __align__(16) uint8_t smem_dyn[];
  uint8_t* sW = smem_dyn;                                                   // staged packed weights, NSTAGE x kQ8StageBytes
  float* sX = reinterpret_cast<float*>(smem_dyn + NSTAGE * kQ8StageBytes);  // [MXC][k/32]
  // the cross-warp reduction buffers reuse the stage slots once every warp is done with them
  float (*sRed)[kQ8Rows][kCols] = reinterpret_cast<float (*)[kQ8Rows][kCols]>(smem_dyn);
  float (*sXt)[kQ8Rows][2][MXC] = reinterpret_cast<float (*)[kQ8Rows][2][MXC]>(smem_dyn + NW * kQ8Rows * kCols * sizeof(float));
  static_assert(NW * kQ8Rows * (kCols + 2 * MXC) * sizeof(float) <= size_t(NSTAGE) * kQ8StageBytes, "reduction buffers must fit");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = warp >> 2, wq = warp & 3, gtid = tid & 127;   // warp group, warp within it, thread within it
  const int g = lane >> 2, t = lane & 3;
  const int r_base = blockIdx.x * kQ8Rows;
  const int nunits = k >> 8, nblk = k >> 5;
  const int nstages = (nunits + kQ8StageUnits - 1) / kQ8StageUnits;
  const int niter = (nstages + SPI - 1) / SPI;
  const int64_t row_bytes = int64_t(nblk) * 34;
  const uint32_t sW_u32 = uint32_t(__cvta_generic_to_shared(sW));

  // Copy assignment inside a warp group: 8 threads per weight row, thread (gtid%8) moves 16-byte chunks
  // (gtid%8) + 8j of the row's 68 chunks per stage.
  const int cp_row = gtid >> 3, cp_c0 = gtid & 7;
  const uint8_t* cp_src = w + int64_t(min(r_base + cp_row, n - 1)) * row_bytes + cp_c0 * 16;
  const uint32_t cp_dst = sW_u32 + cp_row * kQ8Pitch + cp_c0 * 16;
  auto issue_stage = [&](int s) {
    if (s < nstages) {
      const int valid_chunks = min(kQ8StageUnits, nunits - s * kQ8StageUnits) * (kQ8UnitBytes / 16);
      const uint8_t* src = cp_src + int64_t(s) * kQ8StageSrc;
      const uint32_t dst = cp_dst + (s % NSTAGE) * kQ8StageBytes;
#pragma unroll
      for (int j = 0; j < 9; ++j)
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

  // X[c][j] = sum of activations of row c over block j (rows >= m are zero).
  for (int idx = tid; !kOnes && idx < nblk * MXC; idx += NW * 32) {
    const int c = idx / nblk, j = idx - c * nblk;
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
  float xt[MXC];                                   // sum over this lane's (row, block) pairs of d * X
#pragma unroll
  for (int c = 0; c < MXC; ++c) xt[c] = 0.f;
  const int srow = lane >> 1, shalf = lane & 1;    // offset-term role: row lane/2, blocks 4*(lane%2) .. +3 of the unit
  const T* xrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) xrow[nt] = x + int64_t(min(nt * 8 + g, m - 1)) * k + 4 * t;

  for (int it = 0; it < niter; ++it) {
    cp_async_wait<D - 2>();
    __syncthreads();                       // this iteration's stages landed (and X is ready); the previous ones are consumed
    if (it > 0) issue_stage((it - 1 + D) * SPI + grp); else cp_async_commit();
    const int s = it * SPI + grp;
    const int unit = s * kQ8StageUnits + wq;
    if (s < nstages && unit < nunits) {
      const uint8_t* st = sW + (s % NSTAGE) * kQ8StageBytes + wq * kQ8UnitBytes;
      if constexpr (!kOnes) {   // offset term: d * X of four blocks of one row, folded per activation row
        const uint8_t* hb = st + srow * kQ8Pitch + 34 * 4 * shalf;
        float dv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) dv[i] = half_bits_to_float(*reinterpret_cast<const uint16_t*>(hb + 34 * i));
#pragma unroll
        for (int c = 0; c < MXC; ++c) {
          const float4 X = *reinterpret_cast<const float4*>(&sX[c * nblk + unit * 8 + 4 * shalf]);
          xt[c] = fmaf(dv[0], X.x, xt[c]);
          xt[c] = fmaf(dv[1], X.y, xt[c]);
          xt[c] = fmaf(dv[2], X.z, xt[c]);
          xt[c] = fmaf(dv[3], X.w, xt[c]);
        }
      }
      const uint8_t* b0 = st + g * kQ8Pitch;
      const uint8_t* b1 = b0 + 8 * kQ8Pitch;
#pragma unroll
      for (int i = 0; i < 8; ++i) {          // block i of the unit: quants at 34 i + 2, word aligned for odd i
        const T* xp[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) xp[nt] = xrow[nt] + unit * 256 + 32 * i;
        if (i & 1) q8_block<T, NT, MC, false, kOnes>(b0 + 34 * i, b1 + 34 * i, xp, t, res);
        else q8_block<T, NT, MC, true, kOnes>(b0 + 34 * i, b1 + 34 * i, xp, t, res);
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
#pragma unroll
  for (int c = 0; c < MXC; ++c) sXt[warp][srow][shalf][c] = xt[c];
  __syncthreads();
  for (int idx = tid; idx < kQ8Rows * MXC; idx += NW * 32) {
    const int r = idx & (kQ8Rows - 1), c = idx >> 4;
    const int row = r_base + r;
    if (row < n && c < m) {
      float v = 0.f, xs = 0.f;
#pragma unroll
      for (int wv = 0; wv < NW; ++wv) {
        v += sRed[wv][r][c];
        xs += sXt[wv][r][0][c] + sXt[wv][r][1][c];
      }
      v = fmaf(-kOffset, xs, v);
      if (bias != nullptr) v += MT::to_float(bias[row]);
      y[int64_t(c) * n + row] = MT::from_float(v);
    }
  }
}

template <typename T, int MXC, int NW, int NSTAGE>
static int launch_q8_cfg(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, cudaStream_t s) {
  const int tiles = (n + kQ8Rows - 1) / kQ8Rows;
  const size_t smem = size_t(NSTAGE) * kQ8StageBytes + (MXC >= 4 ? 0 : size_t(k / 32) * MXC * sizeof(float));   // the sum table of M <= 2
  if (smem > 200 * 1024) return RC_RANGE;
  auto kern = gemv_q8_0_mma_kernel<T, MXC, NW, NSTAGE>;
  static SmemOptIn granted;             // per kernel instantiation, per device
  if (!smem_opt_in(kern, smem, granted)) return RC_LAUNCH;
  const cudaError_t err = gemv_launch(kern, tiles, 1, NW * 32, smem, s, static_cast<const T*>(a), static_cast<const uint8_t*>(b),
                                      static_cast<const T*>(bias), static_cast<T*>(c), m, n, k);
  return err == cudaSuccess ? RC_OK : RC_LAUNCH;
}

// Few row tiles (all CTAs resident at two per SM): six stage slots per CTA keep more bytes in flight; many row tiles:
// four slots, so that three CTAs fit on an SM (the rule of the Q6_K kernel).
template <typename T, int MXC>
static int launch_q8_m(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, cudaStream_t s) {
  int sm_count = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  if ((n + kQ8Rows - 1) / kQ8Rows <= 2 * sm_count) {
    const int rc = launch_q8_cfg<T, MXC, 8, 6>(a, b, bias, c, m, n, k, s);
    if (rc != RC_RANGE) return rc;
  }
  return launch_q8_cfg<T, MXC, 8, 4>(a, b, bias, c, m, n, k, s);
}

template <typename T>
static int launch_q8(const void* a, const void* b, const void* bias, void* c, int m, int n, int k, cudaStream_t s) {
  if (m == 1) return launch_q8_m<T, 1>(a, b, bias, c, m, n, k, s);
  if (m == 2) return launch_q8_m<T, 2>(a, b, bias, c, m, n, k, s);
  if (m <= 4) return launch_q8_m<T, 4>(a, b, bias, c, m, n, k, s);
  if (m <= 8) return launch_q8_m<T, 8>(a, b, bias, c, m, n, k, s);
  return launch_q8_cfg<T, 16, 4, 3>(a, b, bias, c, m, n, k, s);
}

// K must be a whole number of 256-weight units (rows and units are then 16-byte multiples).
bool gemv_q8_0_mma_supports(int dtype, int m, int k) {
  return (dtype == DINO_BF16 || dtype == DINO_F16) && m >= 1 && m <= 16 && k % 256 == 0;
}

int gemv_q8_0_mma(const void* a, const void* b, const void* bias, void* c, int dtype, int m, int n, int k, cudaStream_t s) {
  return dtype == DINO_BF16 ? launch_q8<__nv_bfloat16>(a, b, bias, c, m, n, k, s) : launch_q8<__half>(a, b, bias, c, m, n, k, s);
}

}  // namespace b200gguf
