/*
 * C ABI of libdinoml_b200_gguf.so - the B200 (sm_100a) implementation of DinoML v2's GGUF
 * quantized-linear path.  Plain pointers and sizes only; every pointer named dev_* / a / b_quant /
 * bias / c is CUDA device memory, `stream` is a cudaStream_t passed as void* (NULL = default stream).
 *
 * Return convention (kernel-level entries): 0 = ok, 1 = null pointer, 2 = non-positive dimension,
 * 3 = k not a multiple of the quantization block (these three follow the reference's fused
 * prototype, kernels/rocm/src/ck_gguf_q8_gemm.hip:1910-1918), 4 = launch failure, 5 = unsupported
 * qtype, 6 = unsupported dtype, 7 = alignment, 8 = shape out of range for the variant, 9 = a bounded
 * device-side wait gave up.  A message for the last failure on the calling thread is available from
 * dino_get_last_error().
 *
 * qtype is the ggml type id the reference stores as `qtype_value` (Q8_0 = 8, Q4_K = 12, Q6_K = 14;
 * src/dinoml/constant_sources.py:88-108; also Q4_0 = 2, Q2_K = 10, Q3_K = 11, Q5_K = 13, MXFP4 = 39, NVFP4 = 40, which the
 * dequantizer and the CUDA-core gemm variant decode).  dtype is a DinoDtype (float16 = 1, float32 = 2,
 * bfloat16 = 6; runtime/include/dinoml/abi.h:14-23).  Activations, bias and output share one dtype,
 * as gemm_rcr requires (src/dinoml/ops/gemm.py:46-60).
 */
#ifndef DINOML_B200_GGUF_H_
#define DINOML_B200_GGUF_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DINOML_B200_GGUF_KERNEL_ABI_VERSION 1

#if defined(__GNUC__)
#define DINOML_B200_API __attribute__((visibility("default")))
#else
#define DINOML_B200_API
#endif

/* Kernel variants of the fused gemm ("candidates" of provider b200_gguf_gemm).  A `variant` argument carries the
 * family in its low byte and a tuning configuration of that family in the second byte (variant | config << 8); config 0
 * is the family's default for the shape.  Configurations exist for STREAM (1 .. dinoml_b200_gguf_variant_configs(4)):
 * consumer warps, ring slots and CTAs per SM of the persistent GEMV - the counterpart of the tile / stage / warp entries
 * of the reference's CUTLASS catalogue (src/dinoml/kernels/providers/cutlass/gemm.py:19-127), ranked by the profiler. */
enum DinoB200GgufVariant {
  DINOML_B200_GGUF_VARIANT_AUTO = 0,   /* shape-guarded dispatch: stream / mma for small M, umma above, simt for float32 */
  DINOML_B200_GGUF_VARIANT_SIMT = 1,   /* CUDA-core warp-per-row, any dtype, any M */
  DINOML_B200_GGUF_VARIANT_MMA = 2,    /* decode GEMV, one CTA per 16-row tile, M = 1..16, float16 / bfloat16; Q8_0, Q4_K, Q6_K */
  DINOML_B200_GGUF_VARIANT_UMMA = 3,   /* prefill GEMM on tcgen05 / TMEM, M >= 9, float16 / bfloat16; every type */
  DINOML_B200_GGUF_VARIANT_STREAM = 4, /* persistent decode GEMV on tensor cores: bulk-copy (TMA) ring + mbarriers, M = 1..8; every type but Q8_0 */
};
#define DINOML_B200_GGUF_VARIANT_CODE(family, config) ((family) | ((config) << 8))

DINOML_B200_API int dinoml_b200_gguf_kernel_abi_version(void);

/* ---- standalone dequantize -------------------------------------------------------------------
 * Replaces libgguf's device entry, same name and argument list as the declaration the reference's
 * generated module carries (src/dinoml/templates/gpu_module.cu.j2:35-42; call site
 * src/dinoml/lowering/ops/gemm.py:745).  dev_in: uint8[rows, n_per_row / block * block_bytes];
 * dev_out: dense [rows, n_per_row]; output_dtype 0 = float32, 1 = float16 (the reference's two),
 * 2 = bfloat16 (extension).  Bit-exact with the reference dequantization arithmetic. */
DINOML_B200_API int libgguf_cuda_dequantize_rows_on_stream(const void* dev_in, int64_t qtype, int64_t rows, int64_t n_per_row,
                                           int output_dtype, void* dev_out, void* stream);

/* ---- fused quantized gemm_rcr[_bias] ----------------------------------------------------------
 * C[m,n] = A[m,k] * dequant(B)[n,k]^T (+ bias[n]).  Fills the slot the reference's dense launcher
 * dinoml_cutlass_gemm_rcr[_bias]_<dtype>_<id>(a, b, [bias,] c, m, n, k, stream) occupies after a
 * dequantize-to-scratch step (src/dinoml/lowering/ops/gemm.py:729-749, src/dinoml/lowering/cuda.py:
 * 205-262), reading the GGUF blocks directly; argument order follows the reference's fused
 * prototype (kernels/rocm/src/ck_gguf_q8_gemm.hip:1910-1940).  bias may be NULL. */
DINOML_B200_API int dinoml_b200_gguf_gemm_rcr(const void* a, const void* b_quant, const void* bias, void* c, int qtype, int dtype,
                              int m, int n, int k, int variant, void* stream);

/* Candidate timer with the contract of the reference's dinoml_profile_cutlass_* symbols
 * (kernels/cuda/src/cutlass_gemm.cu:538-567): one warm launch, then `iterations` launches between two
 * CUDA events on `stream`; returns milliseconds per launch, < 0 on failure. */
DINOML_B200_API float dinoml_profile_b200_gguf_gemm_rcr(const void* a, const void* b_quant, const void* bias, void* c, int qtype,
                                        int dtype, int m, int n, int k, int variant, int iterations, void* stream);

/* Workspace bytes a variant needs for a problem (counterpart of dinoml_cutlass_workspace_*,
 * kernels/cuda/src/cutlass_gemm.cu:1003-1009).  The library keeps such workspace itself, per device. */
DINOML_B200_API size_t dinoml_b200_gguf_gemm_rcr_workspace(int qtype, int dtype, int m, int n, int k, int variant);

/* Which variant AUTO resolves to for a problem (the shape-guarded dispatch the reference emits as
 * if/else text, src/dinoml/lowering/ops/gemm.py:656-698). */
DINOML_B200_API int dinoml_b200_gguf_gemm_rcr_select(int qtype, int dtype, int m, int n, int k);

/* Number of tuning configurations of a variant family (0 for families that have none); valid config values are
 * 1 .. that number.  Counterpart of the length of the reference's per-op candidate list. */
DINOML_B200_API int dinoml_b200_gguf_variant_configs(int family);
/* 1 if the family serves the problem (the predicate the dispatcher and the profiler filter candidates with), else 0. */
DINOML_B200_API int dinoml_b200_gguf_variant_supports(int family, int qtype, int dtype, int m, int n, int k);

/* ---- allocation-free prefill GEMM ---------------------------------------------------------------
 * No counterpart in the reference.  For callers that are not allowed to allocate device memory - a plugin running
 * inside a host that has already handed every byte of HBM to its own arena (so cudaMalloc would fail), or a serving
 * loop that bans cudaMalloc / cudaFree on its hot path because they can stall the whole device.  It is the tensor-core
 * GEMM of dinoml_b200_gguf_gemm_rcr(variant = UMMA) - same shapes (m >= 17, the tcgen05 kernel's weight types, K % 256 == 0, float16 / bfloat16), same
 * arguments minus `variant`, same results - except that its partial tiles (fp32 sums of K ranges that the kernel's
 * stream-K work split cut between SMs) and its flag / status words live in a 16 MiB array plus a 4 KiB one that is part of the library image on every GPU that loads it (dinoml_b200_gguf_prealloc_scratch_bytes()),
 * and that it calls no cudaMalloc, cudaFree or allocating library routine.  The caller still provides a, b_quant,
 * bias and c.  A problem whose partial sums do not fit is refused with code 8 and a message naming both sizes.
 * The first call on each device looks the array's address up (cudaGetSymbolAddress, with that device current); with the
 * CUDA runtime's lazy module loading that is also when the driver places the library's device image (kernel code and these
 * arrays) on that GPU - module loading, not an allocation call, but free device memory drops by the image size then and
 * never again.  Make that first call at start-up, before any stream capture.  All calls on a device share the one array: the kernel
 * overwrites the part it uses before reading it back and lowers every flag it raised, so nothing needs clearing
 * between calls, but two calls that overlap on the GPU (different streams, no dependency) race on it - serialize
 * them. */
DINOML_B200_API int dinoml_b200_gguf_gemm_rcr_prealloc(const void* a, const void* b_quant, const void* bias, void* c, int qtype,
                                                       int dtype, int m, int n, int k, void* stream);
DINOML_B200_API size_t dinoml_b200_gguf_prealloc_scratch_bytes(void);

/* The tcgen05 kernel bounds every barrier wait; a wait that gives up records a code in a per-device
 * status word instead of hanging or trapping.  Synchronizes the device, returns the word (0 = never
 * happened; 1 / 2 / 3 / 4 = a stage-free / stage-ready / accumulator / partial-tile wait gave up; 6 = a peer never signalled
 * in dinoml_b200_peer_exchange; < 0 = CUDA error) and
 * clears it together with the partial-tile flags.
 * No counterpart in the reference. */
DINOML_B200_API int dinoml_b200_gguf_device_status(void);

/* ---- gated dual GEMM on two quantized weights --------------------------------------------------------------------
 * c[M, N] = act(a * dequant(B0)^T) * (a * dequant(B1)^T), act = silu (activation 1) or fast_gelu (2), both products
 * accumulated in fp32, the activation and the product evaluated in fp32, one rounding to `dtype` - the reference's
 * dual_gemm_rcr_silu / dual_gemm_rcr_fast_gelu (src/dinoml/kernels/families/dual_gemm.py:93-103,
 * src/dinoml/lowering/ops/templates/dual_gemm_cpu.cpp.j2:52-75; its CUDA path is a CUTLASS dual GEMM on dense weights,
 * kernels/cuda/src/cutlass_dual_gemm.cu).  Here B0 and B1 are GGUF weights [N, K] of one qtype handed over as ONE
 * buffer `b01_interleaved` of 2N rows in which the rows alternate in groups of 8: rows 16t .. 16t+7 are rows 8t .. 8t+7
 * of B0, rows 16t+8 .. 16t+15 are rows 8t .. 8t+7 of B1 (blocks untouched; a row copy at load time,
 * dinoml_v2_b200.kernels.interleave_rows8).  With that order a gate row and its up row sit in the same thread of the
 * mma GEMV and in lanes l / l^8 of the tcgen05 epilogue, so the gate never goes to memory: one launch for the Llama
 * gate / up pair.  N % 8 == 0; variants stream (M <= 8) and mma (M <= 16) for Q4_K and Q6_K, umma for every type with
 * its usual K / alignment rules; AUTO sends Q8_0 to the umma variant at every M.  Optional extra destinations as in
 * dinoml_b200_gguf_gemm_rcr_scatter (n_peers = 0: none).
 * dinoml_b200_gguf_dual_gemm_rcr_bias is the reference's dual_gemm_rcr_bias_<act> (left_bias_<act>_and_mul,
 * dual_gemm.py:105-135; dual_gemm_cpu.cpp.j2:66-69): c = act(a B0^T + bias0) * (a B1^T + bias1).  `bias01_interleaved`
 * holds 2N values in `dtype`, interleaved in groups of 8 exactly like the rows (8 values of bias0, the 8 matching values
 * of bias1, ...); null = no bias.  A B1 / bias1 of one row ([1, K] broadcast in the reference) is passed as N copies of
 * that row: the host side repeats the row when it builds the interleaved constant. */
DINOML_B200_API int dinoml_b200_gguf_dual_gemm_rcr(const void* a, const void* b01_interleaved, void* c, void* const* peer_c, int n_peers,
                                                   int qtype, int dtype, int m, int n, int k, int activation, int variant, void* stream);
DINOML_B200_API int dinoml_b200_gguf_dual_gemm_rcr_bias(const void* a, const void* b01_interleaved, const void* bias01_interleaved, void* c,
                                                        void* const* peer_c, int n_peers, int qtype, int dtype, int m, int n, int k,
                                                        int activation, int variant, void* stream);

/* ---- sharded decode over peer memory (no counterpart in the reference, which is single-GPU) ----------------------
 * dinoml_b200_gguf_gemv_rcr_scatter: the mma GEMV (M <= 16, Q4_K / Q6_K, float16 / bfloat16; same checks and codes as
 * dinoml_b200_gguf_gemm_rcr with variant = MMA) whose epilogue stores the [M, N] result to `c` AND to `n_peers` (<= 8)
 * further buffers - the same slot of a gather buffer on the other GPUs, mapped into this process (symmetric-memory
 * allocations whose handles the ranks exchange; plain peer stores).  One kernel computes and distributes; there is no separate all-gather.
 * dinoml_b200_gguf_gemm_rcr_scatter: the same for any M - `variant` as in dinoml_b200_gguf_gemm_rcr (AUTO picks mma or
 * umma by shape; shapes only the simt variant serves are refused with code 8).
 * dinoml_b200_peer_exchange: what remains of the collective.  signal_ptrs[r] = the 8-word signal array of rank r
 * (signal_ptrs[rank] is local, zero-initialised once); every rank calls with the same, ever increasing `epoch`.  The
 * kernel publishes "rank's earlier stores are complete" to every peer, waits (bounded, about a second; a rank that
 * never arrives sets device status 6 instead of hanging the GPU) for every peer's signal, and, if count > 0, writes
 * out[i] = sum over r < world of slots[r * count + i] (fp32 accumulation, fixed order): barrier only = all-gather
 * completion, barrier + sum = one-shot all-reduce of GEMV partial results.  A rank leaves the kernel without knowing
 * that its peers finished reading their slots, so do not refill one slot set for the very next exchange: keep two sets and
 * alternate them by epoch parity (dinoml_v2_b200.peer.PeerExchange does), which puts a full barrier between any reader of
 * a set and its next writer.
 * dinoml_b200_peer_exchange_set_poll_limit: polls (200 ns apart) a later exchange makes per peer before it gives up with
 * status 6; 0 restores the default 2^22 (about a second); returns the previous value.
 * dinoml_b200_peer_enable_access: cudaDeviceEnablePeerAccess for the current device towards `peer_device` (success if
 * it was enabled already; code 8 if the GPUs are not peers).  Call it once per peer before passing that GPU's memory
 * to the two entry points above. */
DINOML_B200_API int dinoml_b200_gguf_gemv_rcr_scatter(const void* a, const void* b_quant, const void* bias, void* c, void* const* peer_c,
                                                      int n_peers, int qtype, int dtype, int m, int n, int k, void* stream);
DINOML_B200_API int dinoml_b200_gguf_gemm_rcr_scatter(const void* a, const void* b_quant, const void* bias, void* c, void* const* peer_c,
                                                      int n_peers, int qtype, int dtype, int m, int n, int k, int variant, void* stream);
DINOML_B200_API int dinoml_b200_peer_enable_access(int peer_device);
DINOML_B200_API int dinoml_b200_peer_exchange(void* const* signal_ptrs, int world, int rank, unsigned int epoch, const void* slots,
                                              void* out, int64_t count, int dtype, void* stream);
DINOML_B200_API unsigned int dinoml_b200_peer_exchange_set_poll_limit(unsigned int polls);
/* Pull exchanges for prefill-sized results: the GEMM stores to local memory only, then one kernel (a CTA per SM, 16-byte
 * loads from the peers' buffers over NVLink) does the barrier of dinoml_b200_peer_exchange and moves the data.
 * buffer_ptrs[r] = the (symmetric) buffer of rank r mapped into this process; offsets and sizes in bytes, multiples of 16.
 *   mode 0 (gather): for every p != rank copy bytes [offset + p * chunk_bytes, + chunk_bytes) of rank p's buffer into the
 *     same place of the local buffer - an all-gather of per-rank shards laid out rank-major.
 *   mode 1 (reduce slice): slice `rank` (chunk_bytes) of the sum over ranks r, ascending, fp32, of the partial result that
 *     rank r keeps at offset + r * region_stride of ITS buffer, written to dst_offset + rank * chunk_bytes of the local
 *     buffer.  Followed by a mode-0 call on the result region this is a two-shot all-reduce in which every slice is summed
 *     once, by its owner: identical bits on every rank.
 * Same epoch / reuse rules as dinoml_b200_peer_exchange (each call is one exchange: one epoch). */
DINOML_B200_API int dinoml_b200_peer_pull(void* const* signal_ptrs, void* const* buffer_ptrs, int world, int rank, unsigned int epoch, int mode,
                                          long long offset, long long chunk_bytes, long long region_stride, long long dst_offset, int dtype,
                                          void* stream);
/* The same two kernels with the epoch kept on the DEVICE: `epoch_counter` points to two zero-initialised 32-bit words owned
 * by the caller (one pair per signal array); each launch uses counter + 1 and the last block out stores it back.  For launch
 * sequences captured in a CUDA graph, whose arguments are frozen: every replay still signals a fresh epoch.  Capture an even
 * number of collectives per graph so that the alternation of the two slot sets is the same in every replay. */
DINOML_B200_API int dinoml_b200_peer_exchange_ctr(void* const* signal_ptrs, int world, int rank, unsigned int* epoch_counter, const void* slots,
                                                  void* out, int64_t count, int dtype, void* stream);
DINOML_B200_API int dinoml_b200_peer_pull_ctr(void* const* signal_ptrs, void* const* buffer_ptrs, int world, int rank, unsigned int* epoch_counter,
                                              int mode, long long offset, long long chunk_bytes, long long region_stride, long long dst_offset,
                                              int dtype, void* stream);

/* Per-candidate symbols, named like the reference's kernel symbols so a manifest can carry them:
 *   int   dinoml_b200_gguf_<q>_gemm_rcr_<dtype>_<variant>_v1(a, b_quant, c, m, n, k, stream)
 *   int   dinoml_b200_gguf_<q>_gemm_rcr_bias_<dtype>_<variant>_v1(a, b_quant, bias, c, m, n, k, stream)
 *   float dinoml_profile_b200_gguf_<q>_gemm_rcr_<dtype>_<variant>_v1(a, b_quant, c, m, n, k, iterations, stream)
 * with <q> in {q8_0,q4_k,q6_k} (the six further types q4_0,q5_k,q2_k,q3_k,mxfp4,nvfp4: simt, stream and umma),
 * <dtype> in {float16,bfloat16,float32}, <variant> in {simt,mma,umma,stream}
 * (mma / umma / stream exist for float16 and bfloat16 only; a symbol runs its family's default tuning configuration, the
 * other configurations are reached through dinoml_b200_gguf_gemm_rcr with a variant code). */
#define DINOML_B200_GGUF_DECLARE(q, dt, var)                                                                       \
  DINOML_B200_API int dinoml_b200_gguf_##q##_gemm_rcr_##dt##_##var##_v1(const void* a, const void* b_quant, void* c, int m, int n, \
                                                        int k, void* stream);                                      \
  DINOML_B200_API int dinoml_b200_gguf_##q##_gemm_rcr_bias_##dt##_##var##_v1(const void* a, const void* b_quant, const void* bias, \
                                                             void* c, int m, int n, int k, void* stream);          \
  DINOML_B200_API float dinoml_profile_b200_gguf_##q##_gemm_rcr_##dt##_##var##_v1(const void* a, const void* b_quant, void* c,     \
                                                                  int m, int n, int k, int iterations, void* stream);
#define DINOML_B200_GGUF_DECLARE_Q(q)        \
  DINOML_B200_GGUF_DECLARE(q, float32, simt)  \
  DINOML_B200_GGUF_DECLARE(q, float16, simt)  \
  DINOML_B200_GGUF_DECLARE(q, bfloat16, simt) \
  DINOML_B200_GGUF_DECLARE(q, float16, mma)   \
  DINOML_B200_GGUF_DECLARE(q, bfloat16, mma)  \
  DINOML_B200_GGUF_DECLARE(q, float16, umma)  \
  DINOML_B200_GGUF_DECLARE(q, bfloat16, umma) \
  DINOML_B200_GGUF_DECLARE(q, float16, stream) \
  DINOML_B200_GGUF_DECLARE(q, bfloat16, stream)
DINOML_B200_GGUF_DECLARE_Q(q8_0)
DINOML_B200_GGUF_DECLARE_Q(q4_k)
DINOML_B200_GGUF_DECLARE_Q(q6_k)
/* The six further types of the reference's fused prototype (kernels/rocm/src/ck_gguf_q8_gemm.hip:27-32, 43-69, 80-92; symbol
 * family :1910-1940 per type): dequantize bit-exact; fused gemm on the CUDA-core variant for every dtype, on the persistent
 * GEMV (M <= 8) and the tcgen05 GEMM (M >= 9) for the 16-bit dtypes. */
#define DINOML_B200_GGUF_DECLARE_SIMT_Q(q)    \
  DINOML_B200_GGUF_DECLARE(q, float32, simt)  \
  DINOML_B200_GGUF_DECLARE(q, float16, simt)  \
  DINOML_B200_GGUF_DECLARE(q, bfloat16, simt) \
  DINOML_B200_GGUF_DECLARE(q, float16, stream) \
  DINOML_B200_GGUF_DECLARE(q, bfloat16, stream)
#define DINOML_B200_GGUF_DECLARE_UMMA_Q(q)    \
  DINOML_B200_GGUF_DECLARE(q, float16, umma)  \
  DINOML_B200_GGUF_DECLARE(q, bfloat16, umma)
DINOML_B200_GGUF_DECLARE_UMMA_Q(q4_0)
DINOML_B200_GGUF_DECLARE_UMMA_Q(q5_k)
DINOML_B200_GGUF_DECLARE_UMMA_Q(mxfp4)
DINOML_B200_GGUF_DECLARE_UMMA_Q(nvfp4)
DINOML_B200_GGUF_DECLARE_UMMA_Q(q2_k)
DINOML_B200_GGUF_DECLARE_UMMA_Q(q3_k)
DINOML_B200_GGUF_DECLARE_SIMT_Q(q4_0)
DINOML_B200_GGUF_DECLARE_SIMT_Q(q5_k)
DINOML_B200_GGUF_DECLARE_SIMT_Q(q2_k)
DINOML_B200_GGUF_DECLARE_SIMT_Q(q3_k)
DINOML_B200_GGUF_DECLARE_SIMT_Q(mxfp4)
DINOML_B200_GGUF_DECLARE_SIMT_Q(nvfp4)

/* Last error message of the calling thread ("" if none); same contract as the reference's
 * dino_get_last_error (runtime/src/runtime_common.cpp:5-20). */
DINOML_B200_API const char* dino_get_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* DINOML_B200_GGUF_H_ */
