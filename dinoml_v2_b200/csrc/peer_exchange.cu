// Peer-memory exchange for the sharded (tensor-parallel) decode path: one process per GPU, buffers of every rank mapped
// into every process (symmetric-memory allocations: virtual-memory handles the ranks exchange and map for their own
// GPU), no library collective.
//
// The GEMV kernels store their result into slot [rank] of a gather buffer on EVERY GPU (PeerOut in
// gemv_mma_common.cuh).  What is left of an all-gather is then a barrier, and what is left of an all-reduce is a
// barrier followed by the sum of the `world` slots; this kernel does either:
//   * block 0, thread p != rank:  fence, then store `epoch` into word [rank] of rank p's signal array
//     ("everything this GPU wrote before this kernel is complete");
//   * every block, thread p != rank:  poll word [p] of the local signal array until it reaches `epoch`;
//   * count > 0:  out[i] = sum over r of slots[r][i] (fp32 accumulation, r ascending - identical on every rank).
// The poll is bounded: after `poll_limit` tries (default 2^22, 200 ns apart; peer_exchange_set_poll_limit changes it)
// the kernel records a code in the status word and carries on, so a rank that never arrives cannot hang this GPU.
// Epochs increase by one per call on every rank (host-side counter).
//
// Reuse rule.  A rank leaves this kernel as soon as it has seen every peer's signal for `epoch` and summed its own
// copy of the slots; it does NOT know that the peers have finished reading theirs.  A caller that reused one slot set
// for the very next exchange could therefore overwrite a slow peer's slots while that peer still sums them.  The host
// side (peer.PeerExchange) keeps TWO slot sets and alternates by epoch parity: data for epoch e+1 goes to set (e+1)&1,
// whose last readers ran in exchange e-1, and every rank signalled epoch e only after its exchange e-1 had completed
// (stream order) - so a writer is always a full barrier behind any reader of the set it writes.
//
// The reference has no distributed code; the N-split / K-split scheme this serves is in dinoml_v2_b200/sharding.py.
#include "gemv_mma_common.cuh"

namespace b200gguf {

constexpr uint32_t kPeerSpinLimitDefault = 1u << 22;   // polls, 200 ns apart: about one second
static uint32_t g_peer_poll_limit = kPeerSpinLimitDefault;
enum : int { PEER_ST_TIMEOUT = 6 };

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}

struct PeerSignals {
  uint32_t* ptr[8];       // signal array [8] of every rank, mapped here; ptr[rank] is the local one
};

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }

// Last block out stores the epoch this launch used into the device counter ([0] = epoch, [1] = blocks finished).
__device__ __forceinline__ void advance_epoch(uint32_t* epoch_ctr, uint32_t epoch) {
  if (epoch_ctr == nullptr) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(epoch_ctr + 1, 1u) == gridDim.x - 1) {
      epoch_ctr[1] = 0u;
      __threadfence();
      epoch_ctr[0] = epoch;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
peer_exchange_kernel(const PeerSignals sig, int world, int rank, uint32_t epoch, const T* __restrict__ slots, T* __restrict__ out,
                     int64_t count, int* status, uint32_t poll_limit, uint32_t* epoch_ctr) {
  const int tid = threadIdx.x;
  // Programmatic dependent launch on both sides.  The kernel that follows in the stream (the next GEMV) may start at once:
  // it streams its constant weights while this kernel waits for the peers, and blocks before it reads what this kernel
  // produces.  This kernel itself is resident before its predecessor (the scatter GEMV) has finished and must not
  // publish "my stores are complete" - nor read the slots - until it has.
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  // Device-resident epoch (for launches replayed from a CUDA graph, whose arguments are frozen): every exchange on this
  // counter uses its value + 1 and the last block to finish stores it back.  Read after the dependency wait: every
  // earlier kernel of the stream, the previous exchange included, has completed by then.
  if (epoch_ctr != nullptr) epoch = ld_acquire_sys(epoch_ctr) + 1u;
  if (tid < world && tid != rank) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      st_release_sys(sig.ptr[tid] + rank, epoch);
    }
    bool seen = false;
    for (uint32_t i = 0; i < poll_limit && !seen; ++i) {
      seen = int32_t(ld_acquire_sys(sig.ptr[rank] + tid) - epoch) >= 0;     // wrap-safe "reached"
      if (!seen) __nanosleep(200);
    }
    if (!seen) atomicCAS(status, 0, PEER_ST_TIMEOUT);
  }
  __syncthreads();
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + tid; i < count; i += int64_t(gridDim.x) * blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < world; ++r) acc += to_f32<T>(__ldcg(slots + int64_t(r) * count + i));
    out[i] = from_f32<T>(acc);
  }
  advance_epoch(epoch_ctr, epoch);
}

static __device__ int g_peer_status;
static int* peer_status_ptr() {
  static int* ptr[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_peer_status) != cudaSuccess) return nullptr;
    ptr[dev] = static_cast<int*>(p);
  }
  return ptr[dev];
}

int peer_exchange(void* const* signal_ptrs, int world, int rank, uint32_t epoch, const void* slots, void* out, int64_t count, int dtype,
                  cudaStream_t s, uint32_t* epoch_ctr) {
  if (signal_ptrs == nullptr || world < 1 || world > 8 || rank < 0 || rank >= world) return RC_RANGE;
  if (count < 0 || (count > 0 && (slots == nullptr || out == nullptr))) return RC_NULL;
  int* status = peer_status_ptr();
  if (status == nullptr) return RC_LAUNCH;
  PeerSignals sig;
  for (int i = 0; i < 8; ++i) sig.ptr[i] = i < world ? static_cast<uint32_t*>(signal_ptrs[i]) : nullptr;
  for (int i = 0; i < world; ++i)
    if (sig.ptr[i] == nullptr) return RC_NULL;
  const uint32_t limit = g_peer_poll_limit;
  int64_t blocks = (count + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 64) blocks = 64;
  cudaError_t err = cudaSuccess;
  switch (dtype) {
    case DINO_BF16:
      err = gemv_launch(peer_exchange_kernel<__nv_bfloat16>, int(blocks), 1, 256, 0, s, sig, world, rank, epoch, static_cast<const __nv_bfloat16*>(slots),
                        static_cast<__nv_bfloat16*>(out), count, status, limit, epoch_ctr);
      break;
    case DINO_F16:
      err = gemv_launch(peer_exchange_kernel<__half>, int(blocks), 1, 256, 0, s, sig, world, rank, epoch, static_cast<const __half*>(slots),
                        static_cast<__half*>(out), count, status, limit, epoch_ctr);
      break;
    case DINO_F32:
      err = gemv_launch(peer_exchange_kernel<float>, int(blocks), 1, 256, 0, s, sig, world, rank, epoch, static_cast<const float*>(slots),
                        static_cast<float*>(out), count, status, limit, epoch_ctr);
      break;
    default: return RC_DTYPE;
  }
  return err == cudaSuccess ? RC_OK : RC_LAUNCH;
}

// ---- pull exchanges for large results -----------------------------------------------------------------------------
// For prefill-sized results the scatter epilogue (every CTA storing its tile to every GPU, 2 bytes at a time) is the
// wrong tool; here the GEMM stores to local memory only and one kernel with a CTA per SM moves the data with 16-byte loads
// from the peers' (symmetric) buffers:
//   PULL_GATHER:  after the barrier, copy bytes [p * chunk, (p + 1) * chunk) of region `off` of rank p's buffer into the same
//                 place of the local buffer, for every p != rank.  All-gather of per-rank shards (chunk = shard bytes) and
//                 second half of the all-reduce (chunk = slice bytes of the reduced result).
//   PULL_REDUCE:  after the barrier, out_slice = sum over ranks r (ascending, fp32) of slice `rank` of rank r's partial
//                 result (region `off` + r * region_stride of rank r's buffer), written as slice `rank` of the local
//                 result region `dst_off`.  First half of the all-reduce (reduce-scatter): each slice is summed once, by
//                 its owner, so every rank ends up with identical bits after the gather.
// The barrier is the one of peer_exchange_kernel (publish epoch, poll bounded, status 6 on give-up), run by every CTA.
struct PeerBases {
  uint8_t* ptr[8];        // buffer of every rank, mapped here; ptr[rank] is the local one
};
enum : int { PULL_GATHER = 0, PULL_REDUCE = 1 };

template <typename T>
__global__ void __launch_bounds__(256)
peer_pull_kernel(const PeerSignals sig, const PeerBases base, int world, int rank, uint32_t epoch, int mode, int64_t off, int64_t chunk,
                 int64_t region_stride, int64_t dst_off, int* status, uint32_t poll_limit, uint32_t* epoch_ctr) {
  const int tid = threadIdx.x;
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");          // the GEMM that produced the local data has completed
  if (epoch_ctr != nullptr) epoch = ld_acquire_sys(epoch_ctr) + 1u;
  if (tid < world && tid != rank) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      st_release_sys(sig.ptr[tid] + rank, epoch);
    }
    bool seen = false;
    for (uint32_t i = 0; i < poll_limit && !seen; ++i) {
      seen = int32_t(ld_acquire_sys(sig.ptr[rank] + tid) - epoch) >= 0;
      if (!seen) __nanosleep(200);
    }
    if (!seen) atomicCAS(status, 0, PEER_ST_TIMEOUT);
  }
  __syncthreads();
  const int64_t vecs = chunk >> 4;                               // 16-byte units per chunk (chunk % 16 == 0)
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  if (mode == PULL_GATHER) {
    for (int pi = 1; pi < world; ++pi) {
      const int p = (rank + pi) % world;                         // every rank starts with a different peer
      const uint4* src = reinterpret_cast<const uint4*>(base.ptr[p] + off + int64_t(p) * chunk);
      uint4* dst = reinterpret_cast<uint4*>(base.ptr[rank] + off + int64_t(p) * chunk);
      for (int64_t i = int64_t(blockIdx.x) * blockDim.x + tid; i < vecs; i += stride) dst[i] = __ldcv(src + i);
    }
  } else {
    uint4* dst = reinterpret_cast<uint4*>(base.ptr[rank] + dst_off + int64_t(rank) * chunk);
    constexpr int E = 16 / int(sizeof(T));
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + tid; i < vecs; i += stride) {
      float acc[E];
#pragma unroll
      for (int e = 0; e < E; ++e) acc[e] = 0.f;
      for (int r = 0; r < world; ++r) {
        const uint4 v = __ldcv(reinterpret_cast<const uint4*>(base.ptr[r] + off + int64_t(r) * region_stride + int64_t(rank) * chunk) + i);
        const T* tv = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] += to_f32<T>(tv[e]);
      }
      uint4 o;
      T* to = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int e = 0; e < E; ++e) to[e] = from_f32<T>(acc[e]);
      dst[i] = o;
    }
  }
  advance_epoch(epoch_ctr, epoch);
}

int peer_pull(void* const* signal_ptrs, void* const* buffer_ptrs, int world, int rank, uint32_t epoch, int mode, int64_t off, int64_t chunk,
              int64_t region_stride, int64_t dst_off, int dtype, cudaStream_t s, uint32_t* epoch_ctr) {
  if (signal_ptrs == nullptr || buffer_ptrs == nullptr || world < 1 || world > 8 || rank < 0 || rank >= world) return RC_RANGE;
  if (mode != PULL_GATHER && mode != PULL_REDUCE) return RC_RANGE;
  if (chunk <= 0 || (chunk & 15) || (off & 15) || (dst_off & 15) || (region_stride & 15) || off < 0 || dst_off < 0) return RC_ALIGN;
  int* status = peer_status_ptr();
  if (status == nullptr) return RC_LAUNCH;
  PeerSignals sig;
  PeerBases base;
  for (int i = 0; i < 8; ++i) {
    sig.ptr[i] = i < world ? static_cast<uint32_t*>(signal_ptrs[i]) : nullptr;
    base.ptr[i] = i < world ? static_cast<uint8_t*>(buffer_ptrs[i]) : nullptr;
    if (i < world && (sig.ptr[i] == nullptr || base.ptr[i] == nullptr)) return RC_NULL;
    if (i < world && (reinterpret_cast<uintptr_t>(base.ptr[i]) & 15)) return RC_ALIGN;
  }
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int64_t blocks = (chunk / 16 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 2 * sms) blocks = 2 * sms;
  const uint32_t limit = g_peer_poll_limit;
  cudaError_t err;
  switch (dtype) {
    case DINO_BF16:
      err = gemv_launch(peer_pull_kernel<__nv_bfloat16>, int(blocks), 1, 256, 0, s, sig, base, world, rank, epoch, mode, off, chunk, region_stride,
                        dst_off, status, limit, epoch_ctr);
      break;
    case DINO_F16:
      err = gemv_launch(peer_pull_kernel<__half>, int(blocks), 1, 256, 0, s, sig, base, world, rank, epoch, mode, off, chunk, region_stride, dst_off,
                        status, limit, epoch_ctr);
      break;
    case DINO_F32:
      err = gemv_launch(peer_pull_kernel<float>, int(blocks), 1, 256, 0, s, sig, base, world, rank, epoch, mode, off, chunk, region_stride, dst_off,
                        status, limit, epoch_ctr);
      break;
    default: return RC_DTYPE;
  }
  return err == cudaSuccess ? RC_OK : RC_LAUNCH;
}

// Polls a later exchange makes per peer before it gives up (0 restores the default of 2^22, about a second).  For tests of
// the give-up path and for hosts that want a shorter or longer patience; returns the previous value.
uint32_t peer_exchange_set_poll_limit(uint32_t polls) {
  const uint32_t before = g_peer_poll_limit;
  g_peer_poll_limit = polls == 0 ? kPeerSpinLimitDefault : polls;
  return before;
}

// Lets kernels of the current device load / store memory of `peer_device` (needed before a pointer mapped from another
// GPU is handed to a kernel).  Already enabled counts as success.
int peer_enable_access(int peer_device) {
  int dev = -1, can = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return RC_LAUNCH;
  if (peer_device == dev) return RC_OK;
  if (cudaDeviceCanAccessPeer(&can, dev, peer_device) != cudaSuccess || !can) return RC_RANGE;
  const cudaError_t err = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (err == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return RC_OK; }
  return err == cudaSuccess ? RC_OK : RC_LAUNCH;
}

// Reads (and clears) the exchange status word of the current device.
int peer_device_status() {
  int* status = peer_status_ptr();
  int value = 0;
  if (status == nullptr) return -1;
  if (cudaMemcpy(&value, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (value != 0) cudaMemset(status, 0, sizeof(int));
  return value;
}

}  // namespace b200gguf
