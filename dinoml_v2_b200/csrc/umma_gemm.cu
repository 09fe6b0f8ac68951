// Host side of the tcgen05 prefill GEMM: per-(device, stream) scratch, the stream-K plan, the allocation-free scratch and the
// entry that checks a problem and hands it to the weight type's translation unit.  The kernel is in umma_gemm.cuh.
#include <mutex>
#include <unordered_map>

#include "umma_gemm.cuh"

namespace b200gguf {

namespace umma {

struct DeviceState {
  int* status = nullptr;            // [0] = status word, [1 .. kMaxCtas] = partial-tile flags
  float* workspace = nullptr;
  size_t workspace_bytes = 0;
};
static std::mutex g_mutex;
// One workspace + flag set per (device, stream): launches on one stream are ordered and may share them, launches on
// different streams may overlap on the GPU and must not.
struct StateKey {
  int dev;
  cudaStream_t stream;
  bool operator==(const StateKey& o) const { return dev == o.dev && stream == o.stream; }
};
struct StateKeyHash {
  size_t operator()(const StateKey& k) const { return std::hash<void*>()(static_cast<void*>(k.stream)) * 31u + size_t(k.dev); }
};
static std::unordered_map<StateKey, DeviceState, StateKeyHash> g_state;

static DeviceState* device_state(size_t need_workspace, cudaStream_t stream) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& st = g_state[StateKey{dev, stream}];
  if (st.status == nullptr) {
    if (cudaMalloc(&st.status, sizeof(int) * (1 + kMaxCtas)) != cudaSuccess) return nullptr;
    cudaMemset(st.status, 0, sizeof(int) * (1 + kMaxCtas));
  }
  if (need_workspace > st.workspace_bytes) {
    // Grown outside of stream capture only: callers warm a shape up once before capturing a graph.
    if (st.workspace != nullptr) { cudaDeviceSynchronize(); cudaFree(st.workspace); st.workspace = nullptr; st.workspace_bytes = 0; }
    if (cudaMalloc(&st.workspace, need_workspace) != cudaSuccess) return nullptr;
    st.workspace_bytes = need_workspace;
  }
  return &st;
}

static Plan make_plan(int m, int n, int k) {
  Plan pl;
  pl.bm = m <= 64 ? 64 : m <= 128 ? 128 : 256;
  pl.m_tiles = (m + pl.bm - 1) / pl.bm;
  const long long tiles = static_cast<long long>(pl.m_tiles) * ((n + kRowsW - 1) / kRowsW);
  const int nsb = k / 256;
  pl.units = tiles * nsb;
  int sm_count = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (sm_count > kMaxCtas) sm_count = kMaxCtas;
  // at least four super-blocks per CTA: a small problem is not cut into more pieces than its finishers can add up quickly
  const long long most = pl.units / 4 > 1 ? pl.units / 4 : 1;
  pl.ctas = int(most < sm_count ? most : sm_count);
  pl.workspace_bytes = tiles % pl.ctas == 0 ? 0 : size_t(pl.ctas) * pl.bm * kRowsW * sizeof(float);
  return pl;
}

// ---- allocation-free scratch -------------------------------------------------------------------
// Partial-tile workspace, flags and status word that live in the library's own device image instead of cudaMalloc'ed
// memory.  Every GPU that loads the library carries these 16 MiB until the process exits.
constexpr size_t kStaticScratchBytes = size_t(16) << 20;
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];
static __device__ int g_static_status[1 + kMaxCtas];     // zero-initialised like any static device array

constexpr int kMaxDevices = 64;
struct StaticScratch { float* workspace = nullptr; int* status = nullptr; bool ready = false; };
static StaticScratch g_static[kMaxDevices];

// In host code `g_static_scratch` is only a handle for the symbol, not a device address; the address the kernels
// need is looked up once per device, with that device current.
static int static_scratch(Scratch* out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return RC_LAUNCH;
  std::lock_guard<std::mutex> lock(g_mutex);
  StaticScratch& st = g_static[dev];
  if (!st.ready) {
    void* ws = nullptr;
    void* status = nullptr;
    if (cudaGetSymbolAddress(&ws, g_static_scratch) != cudaSuccess) return RC_LAUNCH;
    if (cudaGetSymbolAddress(&status, g_static_status) != cudaSuccess) return RC_LAUNCH;
    st.workspace = static_cast<float*>(ws);
    st.status = static_cast<int*>(status);
    st.ready = true;
  }
  out->workspace = st.workspace;
  out->status = st.status;
  out->flags = st.status + 1;
  return RC_OK;
}

static int launch_bm(int qtype, int dtype, const void* a, const void* b, const void* bias, void* c, int m, int n, int k, bool use_static,
                     const PeerOut& peers, cudaStream_t s) {
  const Plan pl = make_plan(m, n, k);
  Scratch sc{nullptr, nullptr, nullptr};
  if (use_static) {
    if (pl.workspace_bytes > kStaticScratchBytes) return RC_RANGE;
    if (int rc = static_scratch(&sc)) return rc;
  } else {
    DeviceState* st = device_state(pl.workspace_bytes, s);
    if (st == nullptr) return RC_LAUNCH;
    sc.workspace = st->workspace;
    sc.status = st->status;
    sc.flags = st->status + 1;
  }
  switch (qtype) {
    case QTYPE_Q4_K: return launch_q4_k(dtype, a, b, bias, c, m, n, k, pl, sc, peers, s);
    case QTYPE_Q5_K: return launch_q5_k(dtype, a, b, bias, c, m, n, k, pl, sc, peers, s);
    case QTYPE_Q6_K: return launch_q6_k(dtype, a, b, bias, c, m, n, k, pl, sc, peers, s);
    case QTYPE_Q8_0: return launch_q8_0(dtype, a, b, bias, c, m, n, k, pl, sc, peers, s);
    case QTYPE_Q4_0: return launch_q4_0(dtype, a, b, bias, c, m, n, k, pl, sc, peers, s);
    case QTYPE_MXFP4: return launch_mxfp4(dtype, a, b, bias, c, m, n, k, pl, sc, peers, s);
    case QTYPE_NVFP4: return launch_nvfp4(dtype, a, b, bias, c, m, n, k, pl, sc, peers, s);
    case QTYPE_Q2_K: return launch_q2_k(dtype, a, b, bias, c, m, n, k, pl, sc, peers, s);
    case QTYPE_Q3_K: return launch_q3_k(dtype, a, b, bias, c, m, n, k, pl, sc, peers, s);
    default: return RC_QTYPE;
  }
}

}  // namespace umma

// Packed bytes per 256 weights of a row, 0 for a qtype this kernel does not unpack.
static int super_block_bytes(int qtype) {
  switch (qtype) {
    case QTYPE_Q4_K: case QTYPE_Q4_0: case QTYPE_NVFP4: return 144;
    case QTYPE_Q5_K: return 176;
    case QTYPE_Q6_K: return 210;
    case QTYPE_Q8_0: return 272;
    case QTYPE_MXFP4: return 136;
    case QTYPE_Q2_K: return 84;
    case QTYPE_Q3_K: return 110;
    default: return 0;
  }
}

bool gemm_umma_supports(int qtype, int dtype, int m, int n, int k) {
  (void)n;
  if (super_block_bytes(qtype) == 0 || !(dtype == DINO_BF16 || dtype == DINO_F16) || m < 9 || k % 256 != 0) return false;
  const int64_t row_bytes = int64_t(k / 256) * super_block_bytes(qtype);
  return row_bytes % 16 == 0;   // the packed-weight tensor map needs 16-byte row pitches
}

size_t gemm_umma_workspace(int qtype, int dtype, int m, int n, int k) {
  if (!gemm_umma_supports(qtype, dtype, m, n, k)) return 0;
  return umma::make_plan(m, n, k).workspace_bytes;
}

static int gemm_rcr_umma_impl(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                              bool use_static, const PeerOut& peers, cudaStream_t s) {
  if (int rc = check_gemm_args(a, b, c, qtype, dtype, m, n, k)) return rc;
  if (dtype == DINO_F32) return RC_DTYPE;
  if (super_block_bytes(qtype) == 0) return RC_QTYPE;
  // The kernel walks whole 256-weight super-blocks and derives the weight row pitch from k / 256: a Q8_0 weight whose K
  // is only a multiple of 32 would be misaddressed from the second row on.
  if (k % 256 != 0) return RC_ALIGN;
  if ((reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(a)) & 15) return RC_ALIGN;   // tensor-map bases
  if ((int64_t(k) * 2) & 15) return RC_ALIGN;                       // activation row pitch
  if ((int64_t(k / 256) * super_block_bytes(qtype)) & 15) return RC_ALIGN;   // packed-weight row pitch
  return umma::launch_bm(qtype, dtype, a, b, bias, c, m, n, k, use_static, peers, s);
}

int gemm_rcr_umma(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                  cudaStream_t s) {
  return gemm_rcr_umma_impl(a, b, bias, c, qtype, dtype, m, n, k, false, no_peers(), s);
}

// Same kernel, finished tiles also stored to the extra destinations (see PeerOut).
int gemm_rcr_umma_peers(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                        const PeerOut* peers, cudaStream_t s) {
  return gemm_rcr_umma_impl(a, b, bias, c, qtype, dtype, m, n, k, false, peers != nullptr ? *peers : no_peers(), s);
}

// Same kernel, scratch in the library's static device array: no cudaMalloc / cudaFree anywhere on this path.
int gemm_rcr_umma_static(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                         cudaStream_t s) {
  if (m < 17) return RC_RANGE;   // small M belongs to the GEMV kernels, which need no scratch
  return gemm_rcr_umma_impl(a, b, bias, c, qtype, dtype, m, n, k, true, no_peers(), s);
}
size_t gemm_umma_static_scratch_bytes() { return umma::kStaticScratchBytes; }

// Reads (and clears) the device status word the bounded waits write; 0 = no wait ever gave up.  A launch that gave up
// may have left partial-tile flags raised, so they are cleared with the word.
int umma_device_status() {
  int dev = 0, value = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  std::lock_guard<std::mutex> lock(umma::g_mutex);
  for (auto& entry : umma::g_state) {           // every stream's word on this device; the first non-zero one is reported
    if (entry.first.dev != dev || entry.second.status == nullptr) continue;
    int word = 0;
    if (cudaMemcpy(&word, entry.second.status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (word != 0) {
      cudaMemset(entry.second.status, 0, sizeof(int) * (1 + umma::kMaxCtas));
      if (value == 0) value = word;
    }
  }
  if (dev >= 0 && dev < umma::kMaxDevices && umma::g_static[dev].ready) {   // the static-scratch path's word: always read and cleared
    int word = 0;
    if (cudaMemcpy(&word, umma::g_static[dev].status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (word != 0) {
      cudaMemset(umma::g_static[dev].status, 0, sizeof(int) * (1 + umma::kMaxCtas));
      if (value == 0) value = word;
    }
  }
  return value;
}

}  // namespace b200gguf
