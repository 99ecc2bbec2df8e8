"""Seeded synthetic inputs with the shapes and value distributions of the benchmark workloads.

They stand in for the molecule and crystal datasets the reference trains on (QM9, GEOM-Drugs,
MOF/crystal sets): only sizes and distributions are reproduced, no dataset record.  Everything
is drawn on the CPU from a ``torch.Generator`` so the CPU oracle and the GPU kernels see
identical bits, then moved/cast by the caller.
"""
from __future__ import annotations

import math

import torch


def simplicial_inputs(batch: int, n_max: int, n_lo: int, n_hi: int, heads: int, head_dim: int, scale: float,
                      seed: int = 0, dtype: torch.dtype = torch.float32):  # fmt: skip
    """Padded molecules: atom counts uniform in [n_lo, n_hi], then q,k1,v1,k2,v2 ~ N(0,1)*scale in that
    order, then grad_out ~ N(0,1).  Returns a dict of CPU tensors (heads layout (B,H,N,D))."""
    g = torch.Generator().manual_seed(seed)
    n = torch.randint(n_lo, n_hi + 1, (batch,), generator=g)
    t = {}
    for name in ("q", "k1", "v1", "k2", "v2"):
        t[name] = (torch.randn(batch, heads, n_max, head_dim, generator=g) * scale).to(dtype)
    t["grad_out"] = torch.randn(batch, heads, n_max, head_dim, generator=g).to(dtype)
    valid = torch.arange(n_max)[None, :] < n[:, None]
    t["num_atoms"] = n.to(torch.int32)
    t["valid"] = valid
    return t


def config1(seed: int = 0):
    """B=8, N_max=29, atoms in [9,29], H=8, D=32, fp32, inputs N(0,1)/sqrt(32)."""
    return simplicial_inputs(8, 29, 9, 29, 8, 32, 1.0 / math.sqrt(32.0), seed, torch.float32)


def config2(seed: int = 0, batch: int = 64, dtype: torch.dtype = torch.bfloat16):
    """B=64, N_max=192, atoms in [20,181], H=8, D=64, bf16, inputs N(0,1)/8."""
    return simplicial_inputs(batch, 192, 20, 181, 8, 64, 1.0 / 8.0, seed, dtype)


def simplicial_flops(num_atoms: torch.Tensor, heads: int, head_dim: int) -> dict:
    """Algorithmic FLOPs on valid atoms: forward 4*D*H*sum n^3, backward 10*D*H*sum n^3."""
    s3 = float((num_atoms.double() ** 3).sum())
    return {"fwd": 4.0 * head_dim * heads * s3, "bwd": 10.0 * head_dim * heads * s3,
            "total": 14.0 * head_dim * heads * s3}  # fmt: skip


def random_triclinic_lattices(batch: int, g: torch.Generator, len_lo=15.0, len_hi=30.0, ang_lo=70.0, ang_hi=110.0):
    """(B,6) latents [log a, log b, log c, cos alpha, cos beta, cos gamma]; redraws non-positive-definite cells."""
    out = torch.empty(batch, 6)
    for b in range(batch):
        while True:
            lengths = len_lo + (len_hi - len_lo) * torch.rand(3, generator=g)
            ang = torch.deg2rad(ang_lo + (ang_hi - ang_lo) * torch.rand(3, generator=g))
            ca, cb, cg = torch.cos(ang).tolist()
            if 1.0 - ca * ca - cb * cb - cg * cg + 2.0 * ca * cb * cg > 1e-3:
                break
        out[b, :3] = torch.log(lengths)
        out[b, 3:] = torch.cos(ang)
    return out


def _cell_from_latent(lat: torch.Tensor) -> torch.Tensor:
    from .sparse import lattice_latent_to_cell

    return lattice_latent_to_cell(lat)


def crystal_positions(lattice: torch.Tensor, n: int, g: torch.Generator, min_sep: float = 0.9) -> torch.Tensor:
    """Fractional positions U[0,1)^3 drawn one by one; a draw closer than ``min_sep`` (minimum image over
    27 neighbours) to an accepted atom is rejected."""
    cell = _cell_from_latent(lattice).double()
    B = lattice.shape[0]
    offs = torch.tensor([[i, j, k] for i in (-1, 0, 1) for j in (-1, 0, 1) for k in (-1, 0, 1)], dtype=torch.float64)
    pos = torch.empty(B, n, 3)
    for b in range(B):
        acc = torch.empty(0, 3, dtype=torch.float64)
        while acc.shape[0] < n:
            cand = torch.rand(max(64, n), 3, generator=g).double()
            for c in cand:
                if acc.shape[0] >= n:
                    break
                if acc.shape[0]:
                    d = (c[None, :] - acc)[:, None, :] + offs[None, :, :]
                    r = d @ cell[b]
                    if float(r.square().sum(-1).min()) < min_sep * min_sep:
                        continue
                acc = torch.cat([acc, c[None, :]], 0)
        pos[b] = acc.float()
    return pos


def config3(seed: int = 0, batch: int = 16, n: int = 1024, heads: int = 8, head_dim: int = 64,
            dtype: torch.dtype = torch.bfloat16):  # fmt: skip
    """Periodic crystals: triclinic cells 15-30 A / 70-110 deg, 0.9 A minimum separation, q,k,v ~ N(0,1)/8."""
    g = torch.Generator().manual_seed(seed)
    lat = random_triclinic_lattices(batch, g)
    pos = crystal_positions(lat, n, g)
    t = {"lattice": lat, "pos": pos, "num_atoms": torch.full((batch,), n, dtype=torch.int32), "cutoff": 6.0}
    for name in ("q", "k", "v"):
        t[name] = (torch.randn(batch, heads, n, head_dim, generator=g) / 8.0).to(dtype)
    t["grad_out"] = torch.randn(batch, heads, n, head_dim, generator=g).to(dtype)
    return t


def config4(seed: int = 0, batch: int = 32, n: int = 4096, heads: int = 8, head_dim: int = 64, edge: float = 35.0,
            dtype: torch.dtype = torch.bfloat16, with_qkv: bool = True):  # fmt: skip
    """Cubic cells of edge 35 A with uniform fractional positions; k=16 kNN and window-64 local attention."""
    g = torch.Generator().manual_seed(seed)
    lat = torch.tensor([math.log(edge)] * 3 + [0.0] * 3).repeat(batch, 1)
    pos = torch.rand(batch, n, 3, generator=g)
    t = {"lattice": lat, "pos": pos, "num_atoms": torch.full((batch,), n, dtype=torch.int32), "k": 16, "window": 64}
    if with_qkv:
        for name in ("q", "k_", "v"):
            t[name] = (torch.randn(batch, heads, n, head_dim, generator=g) / 8.0).to(dtype)
        t["grad_out"] = torch.randn(batch, heads, n, head_dim, generator=g).to(dtype)
    return t


ATOM_TYPE_PROBS = (0.51, 0.35, 0.06, 0.07, 0.01)  # H, C, N, O, F


def config5_batch(batch: int, seed: int = 0, n_lo: int = 9, n_hi: int = 29):
    """Small molecules: atom count uniform in [9,29], types from ATOM_TYPE_PROBS, Gaussian positions
    (sigma 1.5 A) with the centre of mass over real atoms removed; padded to the batch maximum."""
    g = torch.Generator().manual_seed(seed)
    n = torch.randint(n_lo, n_hi + 1, (batch,), generator=g)
    n_max = int(n.max())
    valid = torch.arange(n_max)[None, :] < n[:, None]
    types = torch.multinomial(torch.tensor(ATOM_TYPE_PROBS).repeat(batch, 1), n_max, replacement=True, generator=g)
    coords = torch.randn(batch, n_max, 3, generator=g) * 1.5
    coords = coords * valid[..., None]
    com = coords.sum(1, keepdim=True) / n[:, None, None].float()
    coords = (coords - com) * valid[..., None]
    types = types * valid
    return {"atom_types": types, "coords": coords, "pad_mask": ~valid, "num_atoms": n.to(torch.int32)}
