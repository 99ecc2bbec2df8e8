// placeholder until the tcgen05 kernels land
#include "common.cuh"
#include "simplicial.cuh"
namespace mf {
bool simplicial_sm100_supports(int, int, int, int) { return false; }
int simplicial_sm100_fwd(const MfSimplicialFwdArgs&, cudaStream_t) { set_error("tcgen05 path not built"); return MF_ERR_UNSUPPORTED; }
int simplicial_sm100_bwd(const MfSimplicialBwdArgs&, cudaStream_t) { set_error("tcgen05 path not built"); return MF_ERR_UNSUPPORTED; }
size_t simplicial_sm100_fwd_workspace_bytes(const MfSimplicialFwdArgs&) { return 0; }
size_t simplicial_sm100_bwd_workspace_bytes(const MfSimplicialBwdArgs&) { return 0; }
}
