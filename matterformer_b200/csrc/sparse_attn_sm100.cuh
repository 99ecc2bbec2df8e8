// Interface between the C-ABI layer of the sparse attention operators and their tcgen05 kernels
// (sparse_attn_sm100.cu): bf16, head_dim 64, 128-row owner tiles, operands by bulk tensor copies.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/matterformer_b200.h"

namespace mf {

// Whether the tcgen05 kernels can take this call (type, head dimension, size, alignment, tensor-map encoder).
bool sparse_attn_sm100_applies(const MfSparseAttnArgs& a, bool backward);
// `radius` selects the block-list variant, otherwise the band variant.
int sparse_attn_sm100_fwd(const MfSparseAttnArgs& a, bool radius, cudaStream_t stream);
int sparse_attn_sm100_bwd(const MfSparseAttnArgs& a, bool radius, cudaStream_t stream);
// Copies the kernels' status word (0, or MF_ERR_DEVICE_TIMEOUT after a bounded wait expired) to the host; waits for
// the stream.
int sparse_attn_sm100_status(int32_t* host_status, cudaStream_t stream);

}  // namespace mf
