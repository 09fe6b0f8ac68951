// The tcgen05 prefill GEMM's kernels for Q2_K weights (both 16-bit dtypes, three tile heights, with and without extra
// output destinations); one translation unit per weight type so that they compile side by side.
#include "umma_gemm.cuh"

namespace b200gguf {
namespace umma {

int launch_q2_k(B200_UMMA_LAUNCH_ARGS) { return launch_qtype<QTYPE_Q2_K>(dtype, a, b, bias, c, m, n, k, pl, sc, peers, s); }

}  // namespace umma
}  // namespace b200gguf
