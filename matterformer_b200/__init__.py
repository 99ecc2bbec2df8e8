"""B200 (sm_100a) kernels for Matterformer's attention hot path behind the reference's module API."""
from .simplicial import (
    CudaTwoSimplicialAttentionFunction,
    cuda_simplicial_attention_backward,
    cuda_simplicial_attention_forward,
    install,
    uninstall,
    set_backend,
    set_check_status,
    simplicial_attention_cuda,
)
from .batching import AttentionCostBatchSampler, simplicial_tile_steps
from .hostio import HostPipelinedSimplicial
from .sampler import GraphedDenoiser, edm_sample
from .sparse import (
    RadiusBlocks,
    build_radius_blocks,
    cell_grid_dims,
    knn_topk,
    lattice_latent_to_cell,
    local_window_attention,
    radius_block_sparse_attention,
    set_sparse_backend,
    sparse_device_status,
)

__all__ = [
    "GraphedDenoiser",
    "edm_sample",
    "AttentionCostBatchSampler",
    "simplicial_tile_steps",
    "HostPipelinedSimplicial",
    "CudaTwoSimplicialAttentionFunction",
    "cuda_simplicial_attention_backward",
    "cuda_simplicial_attention_forward",
    "install",
    "uninstall",
    "set_backend",
    "set_check_status",
    "simplicial_attention_cuda",
    "RadiusBlocks",
    "build_radius_blocks",
    "cell_grid_dims",
    "knn_topk",
    "lattice_latent_to_cell",
    "local_window_attention",
    "radius_block_sparse_attention",
    "set_sparse_backend",
    "sparse_device_status",
]
