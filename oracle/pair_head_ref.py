"""CPU restatement of the equivariant coordinate head (TEST INFRASTRUCTURE, never imported by the product).

Follows the reference line by line, including the (B, N, N, 2d+16) concatenation the CUDA kernel avoids:
* pair geometry of ``NonPeriodicGeometryAdapter.forward`` (src/matterformer/geometry/adapters.py:83-125),
* ``QM9EDMModel._distance_rbf`` (src/matterformer/models/qm9.py:460-469),
* ``QM9EDMModel._equivariant_coord_delta`` (src/matterformer/models/qm9.py:478-501).

Pinned by ``tests/golden/pair_head.npz``, which ``tests/golden/make_golden.py pair_head`` wrote from the imported
reference model (outputs and gradients).
"""
from __future__ import annotations

import torch


def rbf_constants(n_rbf: int = 16, rbf_max: float = 4.0):
    """Centers and width exactly as the reference registers them (models/qm9.py:448-458)."""
    centers = torch.linspace(0.0, rbf_max, n_rbf, dtype=torch.float32)
    delta = rbf_max / max(n_rbf - 1, 1)
    gamma = torch.tensor(1.0 / max(delta * delta, 1e-6), dtype=torch.float32)
    return centers, gamma


def equivariant_coord_delta(trunk_out, coords, pad_mask, w0, b0, w1, b1, centers, gamma):
    """trunk_out (B,N,d), coords (B,N,3), pad_mask (B,N) bool (True = padding); pair MLP = Linear(w0, b0) -> SiLU ->
    Linear(w1, b1) on cat[h_i, h_j, rbf_ij].  Returns the (B,N,3) coordinate update."""
    coords = coords.float()
    valid = ~pad_mask
    pair_mask = valid[:, :, None] & valid[:, None, :]
    delta = coords[:, :, None, :] - coords[:, None, :, :]
    dist = delta.square().sum(-1).clamp_min(0.0).sqrt()
    sq = coords.square().sum(-1) * valid.to(coords.dtype)
    rms = (sq.sum(1) / valid.sum(1).clamp_min(1)).clamp_min(1e-8).sqrt()
    dist_norm = dist / rms[:, None, None].clamp_min(1e-8)
    delta = delta * pair_mask[..., None]
    dist_norm = dist_norm * pair_mask
    rbf = torch.exp(-gamma * (dist_norm[..., None] - centers.view(1, 1, 1, -1)).square())
    n = trunk_out.shape[1]
    hi = trunk_out[:, :, None, :].expand(-1, -1, n, -1)
    hj = trunk_out[:, None, :, :].expand(-1, n, -1, -1)
    x = torch.cat([hi, hj, rbf.to(trunk_out.dtype)], dim=-1)
    w = torch.nn.functional.linear(torch.nn.functional.silu(torch.nn.functional.linear(x, w0, b0)), w1, b1).squeeze(-1)
    w = w.masked_fill(~pair_mask, 0.0)
    w = w - torch.diag_embed(torch.diagonal(w, dim1=-2, dim2=-1))
    out = (w[..., None] * delta).sum(dim=2)
    denom = valid.to(out.dtype).sum(dim=1, keepdim=True).clamp_min(1.0)
    out = (out / denom.unsqueeze(-1)).masked_fill(pad_mask[..., None], 0.0)
    mean = (out * valid[..., None].to(out.dtype)).sum(dim=1, keepdim=True) / denom.unsqueeze(-1)
    return (out - mean).masked_fill(pad_mask[..., None], 0.0)
