// extern "C" surface of the kernel library: dequantize, fused gemm variants, per-candidate symbols,
// candidate timers.  Declarations (with the reference interfaces they stand in for) are in
// include/dinoml_b200_gguf.h.
#include <string>

#include "../../include/dinoml_b200_gguf.h"
#include "gguf_common.cuh"

namespace b200gguf {

int dequantize_rows(const void* dev_in, int64_t qtype, int64_t rows, int64_t n_per_row, int output_dtype, void* dev_out,
                    cudaStream_t stream);
int gemm_rcr_simt(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                  cudaStream_t s);
int gemm_rcr_mma(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                 cudaStream_t s);
int gemm_rcr_umma(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                  cudaStream_t s);
bool gemv_mma_supports(int qtype, int dtype, int m, int n, int k);
bool gemv_stream_supports(int qtype, int dtype, int m, int n, int k);
int gemv_stream_configs();
int stream_device_status();
bool gemm_umma_supports(int qtype, int dtype, int m, int n, int k);
size_t gemm_umma_workspace(int qtype, int dtype, int m, int n, int k);
int umma_device_status();
int peer_device_status();
int peer_enable_access(int peer_device);
struct PeerOut { void* ptr[8]; int count; int act; };   // layout of gemv_mma_common.cuh
int gemm_rcr_mma_peers(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                       const PeerOut* peer_out, cudaStream_t s);
int gemm_rcr_umma_peers(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                        const PeerOut* peer_out, cudaStream_t s);
int peer_exchange(void* const* signal_ptrs, int world, int rank, uint32_t epoch, const void* slots, void* out, int64_t count, int dtype,
                  cudaStream_t s, uint32_t* epoch_ctr);
uint32_t peer_exchange_set_poll_limit(uint32_t polls);
int peer_pull(void* const* signal_ptrs, void* const* buffer_ptrs, int world, int rank, uint32_t epoch, int mode, int64_t off, int64_t chunk,
              int64_t region_stride, int64_t dst_off, int dtype, cudaStream_t s, uint32_t* epoch_ctr);
int gemm_rcr_stream(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k, int config,
                    cudaStream_t s);
int gemm_rcr_stream_peers(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k, int config,
                          const PeerOut* peer_out, cudaStream_t s);
int gemm_rcr_umma_static(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
                         cudaStream_t s);
size_t gemm_umma_static_scratch_bytes();

// Thread-local last error, same contract as the reference runtime (runtime/src/runtime_common.cpp:5-20).
static thread_local std::string g_last_error;

int set_error(int rc, const char* where) {
  static const char* const kText[] = {
      "ok", "null pointer", "non-positive dimension", "k is not a multiple of the quantization block size",
      "CUDA launch failed", "unsupported GGUF qtype", "unsupported dtype", "pointer or row pitch alignment not met",
      "shape outside the range of this kernel variant", "device-side wait gave up"};
  if (rc == RC_OK) return rc;
  g_last_error = std::string(where) + ": " + (rc > 0 && rc < 10 ? kText[rc] : "error");
  if (rc == RC_LAUNCH) {
    g_last_error += " (";
    g_last_error += cudaGetErrorString(cudaPeekAtLastError());
    g_last_error += ")";
  }
  return rc;
}
int set_error_message(int rc, const std::string& message) {
  g_last_error = message;
  return rc;
}
const char* last_error() { return g_last_error.c_str(); }

int select_variant(int qtype, int dtype, int m, int n, int k) {
  // Shape guard written from measurements on B200 (us per launch, graph replay, cold weights); a profiled execution plan
  // overrides it per shape.
  const int64_t weights = int64_t(n) * k;
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  const int tiles = (n + 15) / 16;
  // M = 8 on a large weight: the tcgen05 kernel costs the same for any M <= 64 and overtakes the GEMVs there
  //   ([8192 x 14336] Q4_K: 27.6 us against 33.9 persistent / 58.2 tile; [4096 x 4096]: 10.4 against 8.9 persistent).
  if (m == 8 && weights >= (int64_t(32) << 20) && (qtype == QTYPE_Q4_K || qtype == QTYPE_Q6_K) && gemm_umma_supports(qtype, dtype, 9, n, k))
    return DINOML_B200_GGUF_VARIANT_UMMA;
  // M <= 8 on Q4_K / Q6_K: the persistent bulk-copy GEMV, except where the tile kernel measured faster:
  //   Q4_K, M = 1, when the tile kernel's grid (three CTAs of 16 rows per SM) fills at least three quarters of its last wave
  //   ([11008 x 4096]: 9.4 us against 10.5 us; with emptier waves or less than one wave the persistent kernel wins);
  //   Q4_K, M >= 2, with fewer row tiles than half the SMs: the tile kernel cuts K across a cluster and so uses more SMs
  //   ([256 x 14336], M = 8: 4.9 us against 9.3 us; [2048 x 4096], M = 8: 6.3 against 5.9);
  //   Q6_K, M >= 3, on weights below 32 M elements ([4096 x 4096], M = 4: 6.3 us against 6.8 us), where the launch is too short
  //   for the ring to pay off (at M <= 2 and on larger weights it is 7 - 30 % faster: [4096 x 14336], M = 1: 15.0 us against 21.1 us).
  if (gemv_stream_supports(qtype, dtype, m, n, k)) {
    bool tile_kernel = false;
    if (qtype == QTYPE_Q4_K && m == 1) {
      const int slots = 3 * sms;
      const int waves = (tiles + slots - 1) / slots;
      // fewer tiles than SMs: the tile kernel on a short K ([1024 x 4096]: 3.1 us against 3.5), the persistent one on a long K,
      // where its ring keeps more bytes in flight per SM ([1024 x 14336]: 7.2 us against 8.9; [256 x 14336]: 7.0 against 8.5)
      tile_kernel = (tiles <= sms && k < 8192) || (tiles >= slots && double(tiles) / (double(waves) * slots) >= 0.75);
    } else if (qtype == QTYPE_Q4_K) {
      // ... on a long K; on K = 4096 the persistent kernel (16 consumer warps per CTA) is ahead from M = 4 since both kernels take
      // their activation sums from the tensor cores ([1024 x 4096], M = 8: 4.6 us against 5.5; [1024 x 14336]: 9.6 against 7.6)
      tile_kernel = 2 * tiles <= sms && (m < 4 || k >= 8192);
    } else if (qtype == QTYPE_Q6_K && m >= 3) {
      tile_kernel = weights < (int64_t(32) << 20);
    }
    // The further types run on tensor cores there too ([4096 x 4096], M = 1 / 8: Q4_0 5.3 / 10.1 us, MXFP4 6.0 / 7.9 us, NVFP4 6.4 / 7.4 us
    // against 15.4 / 32.8, 16.8 / 37.9 and 20.5 / 36.0 on the simt kernel).
    if (!tile_kernel) return DINOML_B200_GGUF_VARIANT_STREAM;
  }
  // M = 9..16 is served by both tensor-core kernels: the tcgen05 one costs the same whatever M is (about 8.5 us at least),
  // the mma.sync GEMV does twice the MMA work of M <= 8.  Crossover by weight size: Q4_K from 4 M elements
  //   ([1024 x 4096], M = 9: 8.6 us against 11.4; [512 x 4096]: 8.5 against 8.3); Q6_K, whose tile kernel is the quicker of the
  //   two, from 32 M elements, or from 8 M at M >= 12 ([4096 x 4096], M = 9: 11.1 us against 9.8, M = 16: 10.8 against 11.3).
  if (m >= 9 && m <= 16 && gemm_umma_supports(qtype, dtype, m, n, k)) {
    const int64_t from = qtype == QTYPE_Q6_K ? (m >= 12 ? int64_t(8) << 20 : int64_t(32) << 20) : int64_t(4) << 20;
    if (weights >= from || !gemv_mma_supports(qtype, dtype, m, n, k)) return DINOML_B200_GGUF_VARIANT_UMMA;
  }
  if (gemv_mma_supports(qtype, dtype, m, n, k)) return DINOML_B200_GGUF_VARIANT_MMA;
  if (gemm_umma_supports(qtype, dtype, m, n, k)) return DINOML_B200_GGUF_VARIANT_UMMA;
  return DINOML_B200_GGUF_VARIANT_SIMT;
}

// A variant code = family (low byte) + tuning configuration (second byte, 0 = the family's default for the shape).
int gemm_rcr(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n, int k,
             int variant, cudaStream_t s) {
  if (variant < 0 || variant > 0xffff) return RC_RANGE;
  const int config = (variant >> 8) & 0xff;
  variant &= 0xff;
  if (variant == DINOML_B200_GGUF_VARIANT_AUTO) variant = select_variant(qtype, dtype, m, n, k);
  if (config != 0 && variant != DINOML_B200_GGUF_VARIANT_STREAM) return RC_RANGE;
  switch (variant) {
    case DINOML_B200_GGUF_VARIANT_STREAM: return gemm_rcr_stream(a, b, bias, c, qtype, dtype, m, n, k, config, s);
    case DINOML_B200_GGUF_VARIANT_SIMT: return gemm_rcr_simt(a, b, bias, c, qtype, dtype, m, n, k, s);
    case DINOML_B200_GGUF_VARIANT_MMA: return gemm_rcr_mma(a, b, bias, c, qtype, dtype, m, n, k, s);
    case DINOML_B200_GGUF_VARIANT_UMMA: return gemm_rcr_umma(a, b, bias, c, qtype, dtype, m, n, k, s);
    default: return RC_RANGE;
  }
}

// Gated dual GEMM on a row-interleaved weight (see dinoml_b200_gguf_dual_gemm_rcr in the header); n = output columns.
// bias01: null, or 2n values in the activation dtype interleaved like the rows (bias0 of 8 gate rows, bias1 of their up rows).
int dual_gemm_rcr_peers(const void* a, const void* b01, const void* bias01, void* c, const PeerOut& dst, int qtype, int dtype, int m, int n,
                        int k, int activation, int variant, cudaStream_t s) {
  if (activation != 1 && activation != 2) return RC_RANGE;
  if (n <= 0 || n % 8 != 0 || n > 0x3fffffff) return RC_RANGE;       // whole groups of 8 rows per matrix
  if (variant < 0 || variant > 0xffff) return RC_RANGE;
  const int config = (variant >> 8) & 0xff;
  variant &= 0xff;
  PeerOut peers = dst;
  peers.act = activation;
  const int rows = 2 * n;                                              // rows of the interleaved weight
  if (variant == DINOML_B200_GGUF_VARIANT_AUTO) {
    variant = select_variant(qtype, dtype, m, rows, k);
    // the Q8_0 mma GEMV has no gated epilogue: the tcgen05 kernel takes the call instead, whatever M is (its 64-row
    // activation tile is zero-filled past M)
    if (variant == DINOML_B200_GGUF_VARIANT_MMA && qtype == QTYPE_Q8_0 && gemm_umma_supports(qtype, dtype, m < 9 ? 9 : m, rows, k))
      variant = DINOML_B200_GGUF_VARIANT_UMMA;
  }
  if (variant == DINOML_B200_GGUF_VARIANT_STREAM) return gemm_rcr_stream_peers(a, b01, bias01, c, qtype, dtype, m, rows, k, config, &peers, s);
  if (config != 0) return RC_RANGE;
  if (variant == DINOML_B200_GGUF_VARIANT_MMA) return gemm_rcr_mma_peers(a, b01, bias01, c, qtype, dtype, m, rows, k, &peers, s);
  if (variant == DINOML_B200_GGUF_VARIANT_UMMA) return gemm_rcr_umma_peers(a, b01, bias01, c, qtype, dtype, m, rows, k, &peers, s);
  return RC_RANGE;                                                     // the simt variant has no gated epilogue
}
int dual_gemm_rcr(const void* a, const void* b01, const void* bias01, void* c, int qtype, int dtype, int m, int n, int k, int activation,
                  int variant, cudaStream_t s) {
  PeerOut none;
  for (int i = 0; i < 8; ++i) none.ptr[i] = nullptr;
  none.count = 0;
  none.act = 0;
  return dual_gemm_rcr_peers(a, b01, bias01, c, none, qtype, dtype, m, n, k, activation, variant, s);
}

float profile_gemm_rcr(const void* a, const void* b, const void* bias, void* c, int qtype, int dtype, int m, int n,
                       int k, int variant, int iterations, cudaStream_t s) {
  if (iterations <= 0) return -1.f;
  if (set_error(gemm_rcr(a, b, bias, c, qtype, dtype, m, n, k, variant, s), "dinoml_profile_b200_gguf_gemm_rcr"))
    return -1.f;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return -1.f;
  float ms = -1.f;
  bool ok = cudaEventRecord(e0, s) == cudaSuccess;
  for (int i = 0; ok && i < iterations; ++i) ok = gemm_rcr(a, b, bias, c, qtype, dtype, m, n, k, variant, s) == RC_OK;
  ok = ok && cudaEventRecord(e1, s) == cudaSuccess && cudaEventSynchronize(e1) == cudaSuccess;
  if (ok && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) ms /= float(iterations); else ms = -1.f;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return ms;
}

}  // namespace b200gguf

using namespace b200gguf;

extern "C" {

int dinoml_b200_gguf_kernel_abi_version(void) { return DINOML_B200_GGUF_KERNEL_ABI_VERSION; }

const char* dino_get_last_error(void) { return last_error(); }

int libgguf_cuda_dequantize_rows_on_stream(const void* dev_in, int64_t qtype, int64_t rows, int64_t n_per_row,
                                           int output_dtype, void* dev_out, void* stream) {
  return set_error(dequantize_rows(dev_in, qtype, rows, n_per_row, output_dtype, dev_out, static_cast<cudaStream_t>(stream)),
                   "libgguf_cuda_dequantize_rows_on_stream");
}

int dinoml_b200_gguf_gemm_rcr(const void* a, const void* b_quant, const void* bias, void* c, int qtype, int dtype, int m,
                              int n, int k, int variant, void* stream) {
  return set_error(gemm_rcr(a, b_quant, bias, c, qtype, dtype, m, n, k, variant, static_cast<cudaStream_t>(stream)),
                   "dinoml_b200_gguf_gemm_rcr");
}

float dinoml_profile_b200_gguf_gemm_rcr(const void* a, const void* b_quant, const void* bias, void* c, int qtype,
                                        int dtype, int m, int n, int k, int variant, int iterations, void* stream) {
  return profile_gemm_rcr(a, b_quant, bias, c, qtype, dtype, m, n, k, variant, iterations, static_cast<cudaStream_t>(stream));
}

size_t dinoml_b200_gguf_gemm_rcr_workspace(int qtype, int dtype, int m, int n, int k, int variant) {
  if (variant == DINOML_B200_GGUF_VARIANT_AUTO) variant = select_variant(qtype, dtype, m, n, k);
  return variant == DINOML_B200_GGUF_VARIANT_UMMA ? gemm_umma_workspace(qtype, dtype, m, n, k) : 0;
}

int dinoml_b200_gguf_gemm_rcr_prealloc(const void* a, const void* b_quant, const void* bias, void* c, int qtype, int dtype,
                                       int m, int n, int k, void* stream) {
  const int rc = gemm_rcr_umma_static(a, b_quant, bias, c, qtype, dtype, m, n, k, static_cast<cudaStream_t>(stream));
  if (rc == RC_RANGE) {
    const size_t need = gemm_umma_workspace(qtype, dtype, m, n, k);
    if (need > gemm_umma_static_scratch_bytes())
      return set_error_message(rc, "dinoml_b200_gguf_gemm_rcr_prealloc: this problem needs " + std::to_string(need) +
                                       " bytes of partial-tile scratch, the built-in scratch holds " +
                                       std::to_string(gemm_umma_static_scratch_bytes()) + "; use dinoml_b200_gguf_gemm_rcr");
  }
  return set_error(rc, "dinoml_b200_gguf_gemm_rcr_prealloc");
}

size_t dinoml_b200_gguf_prealloc_scratch_bytes(void) { return gemm_umma_static_scratch_bytes(); }

int dinoml_b200_gguf_device_status(void) {
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  const int peer = peer_device_status();   // read all three so that all are cleared
  const int gemm = umma_device_status();
  const int gemv = stream_device_status();
  return gemm != 0 ? gemm : gemv != 0 ? gemv : peer;
}

int dinoml_b200_gguf_gemv_rcr_scatter(const void* a, const void* b_quant, const void* bias, void* c, void* const* peer_c, int n_peers,
                                      int qtype, int dtype, int m, int n, int k, void* stream) {
  if (n_peers < 0 || n_peers > 8 || (n_peers > 0 && peer_c == nullptr))
    return set_error(RC_RANGE, "dinoml_b200_gguf_gemv_rcr_scatter");
  PeerOut peers;
  for (int i = 0; i < 8; ++i) peers.ptr[i] = i < n_peers ? peer_c[i] : nullptr;
  peers.count = n_peers;
  peers.act = 0;
  for (int i = 0; i < n_peers; ++i)
    if (peers.ptr[i] == nullptr) return set_error(RC_NULL, "dinoml_b200_gguf_gemv_rcr_scatter");
  return set_error(gemm_rcr_mma_peers(a, b_quant, bias, c, qtype, dtype, m, n, k, &peers, static_cast<cudaStream_t>(stream)),
                   "dinoml_b200_gguf_gemv_rcr_scatter");
}

int dinoml_b200_gguf_gemm_rcr_scatter(const void* a, const void* b_quant, const void* bias, void* c, void* const* peer_c, int n_peers,
                                      int qtype, int dtype, int m, int n, int k, int variant, void* stream) {
  const char* where = "dinoml_b200_gguf_gemm_rcr_scatter";
  if (n_peers < 0 || n_peers > 8 || (n_peers > 0 && peer_c == nullptr)) return set_error(RC_RANGE, where);
  PeerOut peers;
  for (int i = 0; i < 8; ++i) peers.ptr[i] = i < n_peers ? peer_c[i] : nullptr;
  peers.count = n_peers;
  peers.act = 0;
  for (int i = 0; i < n_peers; ++i)
    if (peers.ptr[i] == nullptr) return set_error(RC_NULL, where);
  if (variant < 0 || variant > 0xffff) return set_error(RC_RANGE, where);
  const int config = (variant >> 8) & 0xff;
  variant &= 0xff;
  if (variant == DINOML_B200_GGUF_VARIANT_AUTO) variant = select_variant(qtype, dtype, m, n, k);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (variant == DINOML_B200_GGUF_VARIANT_STREAM)
    return set_error(gemm_rcr_stream_peers(a, b_quant, bias, c, qtype, dtype, m, n, k, config, &peers, s), where);
  if (config != 0) return set_error(RC_RANGE, where);
  if (variant == DINOML_B200_GGUF_VARIANT_MMA) return set_error(gemm_rcr_mma_peers(a, b_quant, bias, c, qtype, dtype, m, n, k, &peers, s), where);
  if (variant == DINOML_B200_GGUF_VARIANT_UMMA) return set_error(gemm_rcr_umma_peers(a, b_quant, bias, c, qtype, dtype, m, n, k, &peers, s), where);
  return set_error(RC_RANGE, where);     // the simt variant has no scatter epilogue
}

int dinoml_b200_gguf_dual_gemm_rcr(const void* a, const void* b01_interleaved, void* c, void* const* peer_c, int n_peers, int qtype,
                                   int dtype, int m, int n, int k, int activation, int variant, void* stream) {
  return dinoml_b200_gguf_dual_gemm_rcr_bias(a, b01_interleaved, nullptr, c, peer_c, n_peers, qtype, dtype, m, n, k, activation, variant, stream);
}

int dinoml_b200_gguf_dual_gemm_rcr_bias(const void* a, const void* b01_interleaved, const void* bias01_interleaved, void* c,
                                        void* const* peer_c, int n_peers, int qtype, int dtype, int m, int n, int k, int activation,
                                        int variant, void* stream) {
  const char* where = "dinoml_b200_gguf_dual_gemm_rcr";
  if (n_peers < 0 || n_peers > 8 || (n_peers > 0 && peer_c == nullptr)) return set_error(RC_RANGE, where);
  PeerOut peers;
  for (int i = 0; i < 8; ++i) peers.ptr[i] = i < n_peers ? peer_c[i] : nullptr;
  peers.count = n_peers;
  peers.act = 0;
  for (int i = 0; i < n_peers; ++i)
    if (peers.ptr[i] == nullptr) return set_error(RC_NULL, where);
  return set_error(dual_gemm_rcr_peers(a, b01_interleaved, bias01_interleaved, c, peers, qtype, dtype, m, n, k, activation, variant,
                                       static_cast<cudaStream_t>(stream)), where);
}

int dinoml_b200_peer_enable_access(int peer_device) {
  return set_error(peer_enable_access(peer_device), "dinoml_b200_peer_enable_access");
}

int dinoml_b200_peer_exchange(void* const* signal_ptrs, int world, int rank, unsigned int epoch, const void* slots, void* out,
                              int64_t count, int dtype, void* stream) {
  return set_error(peer_exchange(signal_ptrs, world, rank, epoch, slots, out, count, dtype, static_cast<cudaStream_t>(stream), nullptr),
                   "dinoml_b200_peer_exchange");
}

int dinoml_b200_peer_exchange_ctr(void* const* signal_ptrs, int world, int rank, unsigned int* epoch_counter, const void* slots, void* out,
                                  int64_t count, int dtype, void* stream) {
  if (epoch_counter == nullptr) return set_error(RC_NULL, "dinoml_b200_peer_exchange_ctr");
  return set_error(peer_exchange(signal_ptrs, world, rank, 0, slots, out, count, dtype, static_cast<cudaStream_t>(stream), epoch_counter),
                   "dinoml_b200_peer_exchange_ctr");
}

unsigned int dinoml_b200_peer_exchange_set_poll_limit(unsigned int polls) { return peer_exchange_set_poll_limit(polls); }

int dinoml_b200_peer_pull(void* const* signal_ptrs, void* const* buffer_ptrs, int world, int rank, unsigned int epoch, int mode, long long offset,
                          long long chunk_bytes, long long region_stride, long long dst_offset, int dtype, void* stream) {
  return set_error(peer_pull(signal_ptrs, buffer_ptrs, world, rank, epoch, mode, offset, chunk_bytes, region_stride, dst_offset, dtype,
                             static_cast<cudaStream_t>(stream), nullptr),
                   "dinoml_b200_peer_pull");
}

int dinoml_b200_peer_pull_ctr(void* const* signal_ptrs, void* const* buffer_ptrs, int world, int rank, unsigned int* epoch_counter, int mode,
                              long long offset, long long chunk_bytes, long long region_stride, long long dst_offset, int dtype, void* stream) {
  if (epoch_counter == nullptr) return set_error(RC_NULL, "dinoml_b200_peer_pull_ctr");
  return set_error(peer_pull(signal_ptrs, buffer_ptrs, world, rank, 0, mode, offset, chunk_bytes, region_stride, dst_offset, dtype,
                             static_cast<cudaStream_t>(stream), epoch_counter),
                   "dinoml_b200_peer_pull_ctr");
}

int dinoml_b200_gguf_gemm_rcr_select(int qtype, int dtype, int m, int n, int k) {
  return select_variant(qtype, dtype, m, n, k);
}

int dinoml_b200_gguf_variant_configs(int family) {
  return family == DINOML_B200_GGUF_VARIANT_STREAM ? gemv_stream_configs() : 0;
}

int dinoml_b200_gguf_variant_supports(int family, int qtype, int dtype, int m, int n, int k) {
  if (qtype_block_size(qtype) == 0 || m <= 0 || n <= 0 || k <= 0 || k % qtype_block_size(qtype) != 0) return 0;
  if (dtype != DINO_F16 && dtype != DINO_BF16 && dtype != DINO_F32) return 0;
  switch (family) {
    case DINOML_B200_GGUF_VARIANT_AUTO:
    case DINOML_B200_GGUF_VARIANT_SIMT: return 1;
    case DINOML_B200_GGUF_VARIANT_MMA: return gemv_mma_supports(qtype, dtype, m, n, k) ? 1 : 0;
    case DINOML_B200_GGUF_VARIANT_UMMA: return gemm_umma_supports(qtype, dtype, m, n, k) ? 1 : 0;
    case DINOML_B200_GGUF_VARIANT_STREAM: return gemv_stream_supports(qtype, dtype, m, n, k) ? 1 : 0;
    default: return 0;
  }
}

#define B200_DEFINE(q, QT, dt, DT, var, VAR)                                                                          \
  int dinoml_b200_gguf_##q##_gemm_rcr_##dt##_##var##_v1(const void* a, const void* b_quant, void* c, int m, int n,    \
                                                        int k, void* stream) {                                        \
    return set_error(gemm_rcr(a, b_quant, nullptr, c, QT, DT, m, n, k, VAR, static_cast<cudaStream_t>(stream)),       \
                     "dinoml_b200_gguf_" #q "_gemm_rcr_" #dt "_" #var "_v1");                                         \
  }                                                                                                                   \
  int dinoml_b200_gguf_##q##_gemm_rcr_bias_##dt##_##var##_v1(const void* a, const void* b_quant, const void* bias,    \
                                                             void* c, int m, int n, int k, void* stream) {            \
    if (bias == nullptr) return set_error(RC_NULL, "dinoml_b200_gguf_" #q "_gemm_rcr_bias_" #dt "_" #var "_v1");      \
    return set_error(gemm_rcr(a, b_quant, bias, c, QT, DT, m, n, k, VAR, static_cast<cudaStream_t>(stream)),          \
                     "dinoml_b200_gguf_" #q "_gemm_rcr_bias_" #dt "_" #var "_v1");                                    \
  }                                                                                                                   \
  float dinoml_profile_b200_gguf_##q##_gemm_rcr_##dt##_##var##_v1(const void* a, const void* b_quant, void* c, int m, \
                                                                  int n, int k, int iterations, void* stream) {       \
    return profile_gemm_rcr(a, b_quant, nullptr, c, QT, DT, m, n, k, VAR, iterations,                                 \
                            static_cast<cudaStream_t>(stream));                                                       \
  }
#define B200_DEFINE_Q(q, QT)                                                              \
  B200_DEFINE(q, QT, float32, DINO_F32, simt, DINOML_B200_GGUF_VARIANT_SIMT)              \
  B200_DEFINE(q, QT, float16, DINO_F16, simt, DINOML_B200_GGUF_VARIANT_SIMT)              \
  B200_DEFINE(q, QT, bfloat16, DINO_BF16, simt, DINOML_B200_GGUF_VARIANT_SIMT)            \
  B200_DEFINE(q, QT, float16, DINO_F16, mma, DINOML_B200_GGUF_VARIANT_MMA)                \
  B200_DEFINE(q, QT, bfloat16, DINO_BF16, mma, DINOML_B200_GGUF_VARIANT_MMA)              \
  B200_DEFINE(q, QT, float16, DINO_F16, umma, DINOML_B200_GGUF_VARIANT_UMMA)              \
  B200_DEFINE(q, QT, bfloat16, DINO_BF16, umma, DINOML_B200_GGUF_VARIANT_UMMA)            \
  B200_DEFINE(q, QT, float16, DINO_F16, stream, DINOML_B200_GGUF_VARIANT_STREAM)          \
  B200_DEFINE(q, QT, bfloat16, DINO_BF16, stream, DINOML_B200_GGUF_VARIANT_STREAM)
B200_DEFINE_Q(q8_0, QTYPE_Q8_0)
B200_DEFINE_Q(q4_k, QTYPE_Q4_K)
B200_DEFINE_Q(q6_k, QTYPE_Q6_K)
// the further types: CUDA-core kernel, persistent GEMV and tcgen05 GEMM for all six
#define B200_DEFINE_SIMT_Q(q, QT)                                                         \
  B200_DEFINE(q, QT, float32, DINO_F32, simt, DINOML_B200_GGUF_VARIANT_SIMT)              \
  B200_DEFINE(q, QT, float16, DINO_F16, simt, DINOML_B200_GGUF_VARIANT_SIMT)              \
  B200_DEFINE(q, QT, bfloat16, DINO_BF16, simt, DINOML_B200_GGUF_VARIANT_SIMT)            \
  B200_DEFINE(q, QT, float16, DINO_F16, stream, DINOML_B200_GGUF_VARIANT_STREAM)          \
  B200_DEFINE(q, QT, bfloat16, DINO_BF16, stream, DINOML_B200_GGUF_VARIANT_STREAM)
#define B200_DEFINE_UMMA_Q(q, QT)                                                         \
  B200_DEFINE(q, QT, float16, DINO_F16, umma, DINOML_B200_GGUF_VARIANT_UMMA)              \
  B200_DEFINE(q, QT, bfloat16, DINO_BF16, umma, DINOML_B200_GGUF_VARIANT_UMMA)
B200_DEFINE_UMMA_Q(q4_0, QTYPE_Q4_0)
B200_DEFINE_UMMA_Q(q5_k, QTYPE_Q5_K)
B200_DEFINE_UMMA_Q(mxfp4, QTYPE_MXFP4)
B200_DEFINE_UMMA_Q(nvfp4, QTYPE_NVFP4)
B200_DEFINE_UMMA_Q(q2_k, QTYPE_Q2_K)
B200_DEFINE_UMMA_Q(q3_k, QTYPE_Q3_K)
B200_DEFINE_SIMT_Q(q4_0, QTYPE_Q4_0)
B200_DEFINE_SIMT_Q(q5_k, QTYPE_Q5_K)
B200_DEFINE_SIMT_Q(q2_k, QTYPE_Q2_K)
B200_DEFINE_SIMT_Q(q3_k, QTYPE_Q3_K)
B200_DEFINE_SIMT_Q(mxfp4, QTYPE_MXFP4)
B200_DEFINE_SIMT_Q(nvfp4, QTYPE_NVFP4)

}  // extern "C"
