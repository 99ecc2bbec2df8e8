"""CPU restatement of the reference primitives that define radius / local-window attention and the
periodic distances (TEST INFRASTRUCTURE; never imported by the product package).

* :func:`lattice_to_cell` / :func:`periodic_pair_dist2` restate
  ``lattice_latent_to_lower_triangular`` (src/matterformer/geometry/lattice.py:12-47) and
  ``PeriodicGeometryAdapter.forward`` (src/matterformer/geometry/adapters.py:176-190): 27 offsets in
  ``itertools.product`` order, ``delta^T G delta`` by einsum with ``G = L L^T``, argmin, clamp >= 0.
* :func:`masked_attention` restates the masked softmax attention ``RotaryMultiheadAttention.forward``
  computes (src/matterformer/models/regular_attention.py:251-268): additive 0 / finfo.min mask handed
  to ``F.scaled_dot_product_attention`` with the default scale ``D^-1/2``.

The reference has no radius or local-window operator; the masks (distance <= cutoff with self
included; band i-w/2 <= j <= i+w/2-1) are this project's definitions, so parity for those two
operators is pinned only through these primitives ("parity unpinned" by reference tests).
"""
from __future__ import annotations

from itertools import product

import torch
import torch.nn.functional as F


def lattice_to_cell(lattice: torch.Tensor) -> torch.Tensor:
    lat = lattice.float()
    log_len = lat[:, :3].clamp(min=-5.0, max=5.0)
    cos = lat[:, 3:].clamp(min=-0.9999, max=0.9999)
    length = torch.exp(log_len)
    ca, cb, cg = cos.unbind(dim=-1)
    sg = torch.sqrt((1.0 - cg.square()).clamp_min(1e-8))
    cell = torch.zeros(lat.shape[0], 3, 3)
    cell[:, 0, 0] = length[:, 0]
    cell[:, 1, 0] = length[:, 1] * cg
    cell[:, 1, 1] = length[:, 1] * sg
    cell[:, 2, 0] = length[:, 2] * cb
    cell[:, 2, 1] = length[:, 2] * (ca - cb * cg) / sg
    cell[:, 2, 2] = torch.sqrt(length[:, 2].square() - cell[:, 2, 0].square() - cell[:, 2, 1].square()).clamp_min(1e-8)
    return cell


def periodic_pair_dist2(frac: torch.Tensor, lattice: torch.Tensor) -> torch.Tensor:
    """(B,N,N) squared minimum-image distances, evaluated the way the reference adapter does."""
    frac = frac.float()
    cell = lattice_to_cell(lattice)
    gram = torch.matmul(cell, cell.transpose(-1, -2))
    offs = torch.tensor(list(product(range(-1, 2), repeat=3)), dtype=torch.float32).view(1, 1, 1, 27, 3)
    out = []
    for b in range(frac.shape[0]):
        delta = frac[b : b + 1, :, None, :] - frac[b : b + 1, None, :, :]
        images = delta[:, :, :, None, :] + offs
        d2 = torch.einsum("bnmki,bij,bnmkj->bnmk", images, gram[b : b + 1], images)
        idx = d2.argmin(dim=-1, keepdim=True)
        out.append(torch.gather(d2, -1, idx).squeeze(-1).clamp_min(0.0))
    return torch.cat(out, 0)


def knn_from_dist2(d2: torch.Tensor, num_atoms: torch.Tensor, k: int, include_self: bool = False):
    """Stable ascending sort of each row of (B,N,N) distances, first k; ties -> lower index."""
    B, N, _ = d2.shape
    d2 = d2.clone()
    valid = torch.arange(N)[None, :] < num_atoms[:, None]
    d2 = d2.masked_fill(~valid[:, None, :], float("inf"))
    if not include_self:
        d2 = d2 + torch.diag_embed(torch.full((B, N), float("inf")))
    val, idx = torch.sort(d2, dim=-1, stable=True)
    idx = idx[..., :k].to(torch.int32)
    val = val[..., :k]
    idx = torch.where(torch.isinf(val), torch.full_like(idx, -1), idx)
    idx = torch.where(valid[:, :, None], idx, torch.full_like(idx, -1))
    val = torch.where(valid[:, :, None], val, torch.full_like(val, float("inf")))
    return idx, val


def masked_attention(q, k, v, visible: torch.Tensor, *, fp32: bool = True) -> torch.Tensor:
    """softmax(q k^T D^-1/2 + mask) v with mask = 0 where ``visible`` (B,N,N) else finfo.min."""
    if fp32:
        q, k, v = q.float(), k.float(), v.float()
    bias = torch.zeros(visible.shape, dtype=q.dtype).masked_fill(~visible, torch.finfo(q.dtype).min)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=bias[:, None, :, :])


def radius_visible(frac, lattice, num_atoms, cutoff: float) -> torch.Tensor:
    d = torch.sqrt(periodic_pair_dist2(frac, lattice))
    N = frac.shape[1]
    valid = torch.arange(N)[None, :] < num_atoms[:, None]
    return (d <= cutoff) & valid[:, :, None] & valid[:, None, :]


def band_visible(n_tokens: int, num_atoms: torch.Tensor, window: int) -> torch.Tensor:
    i = torch.arange(n_tokens)[:, None]
    j = torch.arange(n_tokens)[None, :]
    band = (j >= i - window // 2) & (j <= i + window // 2 - 1)
    valid = torch.arange(n_tokens)[None, :] < num_atoms[:, None]
    return band[None] & valid[:, :, None] & valid[:, None, :]
