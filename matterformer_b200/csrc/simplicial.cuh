// Internal interfaces between the C-ABI layer and the simplicial-attention kernels.
#pragma once

#include <cuda_runtime.h>

#include "../../include/matterformer_b200.h"

namespace mf {

// fp32 CUDA-core kernels (simplicial_generic.cu)
int simplicial_generic_fwd(const MfSimplicialFwdArgs& a, cudaStream_t stream);
int simplicial_generic_bwd(const MfSimplicialBwdArgs& a, cudaStream_t stream);
size_t simplicial_generic_bwd_workspace_bytes(const MfSimplicialBwdArgs& a);

// tcgen05 tensor-core kernels (simplicial_sm100.cu)
bool simplicial_sm100_supports(int dtype, int precision, int tokens, int head_dim);
// Molecules of at most 32 tokens: four heads share one 128-row tile (needs a multiple of four heads).
inline bool simplicial_sm100_packs_heads(int tokens, int heads) { return tokens <= 32 && heads % 4 == 0; }
int simplicial_sm100_fwd(const MfSimplicialFwdArgs& a, cudaStream_t stream);
int simplicial_sm100_bwd(const MfSimplicialBwdArgs& a, cudaStream_t stream);
// Same kernels with rows that are not (B,H,N,D) contiguous (NULL = contiguous); see RowLayout.
struct TileLayouts;
int simplicial_sm100_fwd_layouts(const MfSimplicialFwdArgs& a, const TileLayouts* layouts, cudaStream_t stream);
int simplicial_sm100_bwd_layouts(const MfSimplicialBwdArgs& a, const TileLayouts* layouts, cudaStream_t stream);
size_t simplicial_sm100_fwd_workspace_bytes(const MfSimplicialFwdArgs& a);
size_t simplicial_sm100_bwd_workspace_bytes(const MfSimplicialBwdArgs& a);

// row-packed tcgen05 kernels (simplicial_rows_fwd.cu, simplicial_rows_bwd.cu); same problems as the kernels above
int simplicial_rows_fwd(const MfSimplicialFwdArgs& a, cudaStream_t stream);
int simplicial_rows_bwd(const MfSimplicialBwdArgs& a, cudaStream_t stream);
size_t simplicial_rows_bwd_workspace_bytes(const MfSimplicialBwdArgs& a);

}  // namespace mf
