// Pieces shared by the mma.sync decode GEMV kernels (Q4_K, Q6_K): operand types, cp.async helpers.
#pragma once
#include <mutex>

#include "gguf_common.cuh"

namespace b200gguf {

template <typename T> struct MmaType;
template <> struct MmaType<__nv_bfloat16> {
  static constexpr uint32_t kMagicBytes = 0x43434343u;  // bf16 0x43qq = 128 + q
  static constexpr uint32_t kOnePair = 0x3F803F80u;     // (1.0, 1.0)
  static constexpr float kMagic = 128.f;                // offset left in the MMA operand
  static __device__ __forceinline__ uint32_t fix(uint32_t pair) { return pair; }
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  // d = a * b + c with the C tuple in four registers of its own (a CTA-lifetime quad of zeros: no accumulator to clear)
  static __device__ __forceinline__ void mma_c(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, const float (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
  }
  static __device__ __forceinline__ float2 pair_to_float2(uint32_t r) {   // two packed 16-bit values -> two floats (exact)
    return make_float2(__uint_as_float(r << 16), __uint_as_float(r & 0xffff0000u));
  }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float sum8(const uint4& v) {
    const uint32_t r[4] = {v.x, v.y, v.z, v.w};
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) s += __uint_as_float(r[i] << 16) + __uint_as_float(r[i] & 0xffff0000u);
    return s;
  }
};
template <> struct MmaType<__half> {
  static constexpr uint32_t kMagicBytes = 0x64646464u;  // fp16 0x64qq = 1024 + q ...
  static constexpr uint32_t kOnePair = 0x3C003C00u;     // (1.0, 1.0)
  static constexpr float kMagic = 0.f;                  // ... and the 1024 is removed exactly before the MMA
  static __device__ __forceinline__ uint32_t fix(uint32_t pair) {
    const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&pair), __half2half2(__ushort_as_half(0x6400)));
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ void mma_c(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, const float (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
  }
  static __device__ __forceinline__ float2 pair_to_float2(uint32_t r) { return __half22float2(*reinterpret_cast<const __half2*>(&r)); }
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float sum8(const uint4& v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); s += f.x + f.y; }
    return s;
  }
};

// Four registers holding 0.f whose contents the compiler cannot see through: a stable zero C tuple for mma_c.
__device__ __forceinline__ void opaque_zero4(float (&z)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) asm volatile("mov.f32 %0, 0f00000000;\n" : "=f"(z[i]));
}

// Byte -> float without I2F: 0x4B0000bb is 2^23 + bb.
__device__ __forceinline__ float byte_to_float(uint32_t word, int i) {
  return __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7650 + i)) - 8388608.f;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
// 16-byte shared-memory destination of which only the first `bytes` (1..15) are read from global memory; the rest is
// zero-filled.  Used where a 16-byte chunk would cross the end of the weight buffer.
__device__ __forceinline__ void cp_async16_partial(uint32_t dst, const void* src, int bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// ---- K-split across a thread-block cluster.  grid.y = cluster size = number of K slices of one 16-row tile; the
// slices' partial sums meet in the rank-0 CTA through distributed shared memory (no workspace, fixed summation order).
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float* local, uint32_t rank) {   // the same variable in CTA `rank`
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(uint32_t(__cvta_generic_to_shared(local))), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// K slices per row tile: a CTA should own at most `slots` stages (then all of its bytes are in flight from its first
// instruction on), and a launch with few row tiles is cut further until the machine holds about two CTAs per SM.
// Clusters of up to 8 CTAs are portable.
inline int gemv_k_slices(int tiles, int nstages, int slots) {
  int ks = (nstages + slots - 1) / slots;
  int sm_count = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  while (ks < 8 && tiles * ks < 2 * sm_count && (nstages + ks - 1) / ks > 1) ++ks;
  if (ks > 8) ks = 8;
  if (ks > nstages) ks = nstages;
  return ks < 1 ? 1 : ks;
}

// Extra destinations of a GEMV result: up to 8 more [M, N] buffers (typically the same slot of a gather buffer in
// every peer GPU's memory, mapped into this process) that receive the same values as the primary output, written
// by the same threads with plain stores.  count = 0: none.
struct PeerOut {
  void* ptr[8];
  int count;
  int act;      // 0: plain output.  1 / 2: gated output silu(g) * u / fast_gelu(g) * u of a weight whose rows interleave the
                // two matrices in groups of 8 (rows 16t..16t+7 = rows 8t..8t+7 of the first, 16t+8..16t+15 = of the second)
};
inline PeerOut no_peers() {
  PeerOut p;
  for (int i = 0; i < 8; ++i) p.ptr[i] = nullptr;
  p.count = 0;
  p.act = 0;
  return p;
}
enum : int { ACT_NONE = 0, ACT_SILU = 1, ACT_FAST_GELU = 2 };
// left activation of the reference's dual GEMM (src/dinoml/lowering/ops/templates/dual_gemm_cpu.cpp.j2:66-70), in fp32
__device__ __forceinline__ float gate_activation(float g, int act) {
  if (act == ACT_SILU) return g / (1.0f + expf(-g));
  return 0.5f * g * (1.0f + tanhf(0.7978845608f * g * (1.0f + 0.044715f * g * g)));
}

// Opt-in for more than 48 KB of dynamic shared memory.  cudaFuncSetAttribute applies to the current device only, so the
// largest size already granted is remembered per device (one SmemOptIn per kernel instantiation), under a lock.
constexpr int kGemvMaxDevices = 64;
struct SmemOptIn { size_t bytes[kGemvMaxDevices] = {}; };
inline std::mutex& smem_opt_in_mutex() {
  static std::mutex m;
  return m;
}
template <typename Kernel>
inline bool smem_opt_in(Kernel kern, size_t smem, SmemOptIn& granted) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lock(smem_opt_in_mutex());
  const bool tracked = dev >= 0 && dev < kGemvMaxDevices;
  if (tracked && smem <= granted.bytes[dev]) return true;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return false;
  if (tracked) granted.bytes[dev] = smem;
  return true;
}

// Launch with programmatic stream serialization and, for ks > 1, clusters of ks CTAs along grid.y.
template <typename Kernel, typename... Args>
inline cudaError_t gemv_launch(Kernel kern, int tiles, int ks, int threads, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles, ks);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 1;
  attr[1].val.clusterDim.y = unsigned(ks);
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ks > 1 ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

}  // namespace b200gguf
