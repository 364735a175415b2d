// placeholder until the tcgen05 kernel lands
#include "common.cuh"
#include "conv_dispatch.h"
namespace tsb {
bool igemm_umma_supported(const IgemmArgs&) { return false; }
size_t igemm_umma_workspace_bytes(int, int, int, int) { return 256; }
int igemm_umma(const IgemmArgs&, cudaStream_t) { return TSB_ERR_UNSUPPORTED; }
}  // namespace tsb
