// Pieces shared by the persistent ("stream") decode GEMV kernels: mbarrier helpers with bounded waits, the 1-D bulk
// copy (TMA) wrapper, the per-CTA work split and the status word that records a wait that gave up.
//
// Shape of a stream kernel.  One CTA per SM (or two), each owning a contiguous range of 16-row weight tiles for the
// whole launch.  One producer lane walks that range and stages (16 rows x KC super-blocks) of PACKED bytes with one
// cp.async.bulk per row into a ring of D shared-memory slots, each guarded by a full / empty mbarrier pair; the ring
// keeps running across tile boundaries, so HBM requests never drain between tiles.  Consumer warps wait on mbarriers
// only (no CTA-wide barrier in the loop), keep the exact-integer mma.sync arithmetic of the tile kernels, and hand
// their per-tile partial sums to one epilogue warp through a double-buffered shared-memory area (again mbarriers), so
// they move on to the next tile without waiting for the output to be written.
// Bulk copies are plain: sources are this GPU's weight buffer only, no cluster multicast anywhere.
#pragma once
#include "gemv_mma_common.cuh"

namespace b200gguf {
namespace stream {

constexpr uint64_t kWaitLimitNs = 2000000000ull;   // a wait gives up after two seconds of wall time ...
constexpr uint32_t kSpinLimit = 1u << 28;           // ... or this many polls, whichever comes first
enum : int { ST_STREAM_FULL = 11, ST_STREAM_EMPTY = 12, ST_STREAM_RED_FULL = 13, ST_STREAM_RED_EMPTY = 14, ST_STREAM_PARTIAL = 15 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false - after recording `code` in the status word and raising the CTA's abort flag - if the
// phase does not complete within the limit, or as soon as another role has raised the abort flag.
// The slow path is kept out of line: the loops that call it stay small in the instruction cache.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  const uint64_t start = globaltimer_ns();
  for (uint32_t i = 1; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 0u) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - start > kWaitLimitNs) break;
      __nanosleep(32);
    }
  }
  *abort_flag = 1;
  atomicCAS(status, 0, code);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag, status, code);
}
// Bounded wait with no flagging, for the teardown path (outstanding copies must land before the CTA may exit).
__device__ __forceinline__ void mbar_wait_plain(uint32_t bar, uint32_t parity) {
  const uint64_t start = globaltimer_ns();
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return;
    if ((i & 63u) == 63u) {
      if (globaltimer_ns() - start > kWaitLimitNs) return;
      __nanosleep(64);
    }
  }
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.  dst, src and bytes are
// multiples of 16.  No multicast.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) { asm volatile("st.release.gpu.global.s32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory");
}

// First tile of CTA c when `tiles` row tiles are dealt to `ctas` CTAs in contiguous, near-equal ranges.
__host__ __device__ inline int tile_begin(int c, int tiles, int ctas) { return int((int64_t(c) * tiles) / ctas); }

// Status word of the stream kernels on the current device (a static device variable of the library; 0 = no wait ever
// gave up).  Defined in gemv_stream.cu.
int* stream_status_ptr();

}  // namespace stream
}  // namespace b200gguf
