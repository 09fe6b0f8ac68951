// placeholder until the tcgen05 kernel lands
#include "gguf_common.cuh"
namespace b200gguf {
bool gemm_umma_supports(int, int, int, int, int) { return false; }
size_t gemm_umma_workspace(int, int, int, int, int) { return 0; }
int gemm_rcr_umma(const void*, const void*, const void*, void*, int, int, int, int, int, cudaStream_t) { return RC_RANGE; }
}
