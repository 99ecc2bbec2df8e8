"""Periodic kNN, radius block lists, radius block-sparse attention and local-window attention.

The reference's active package has no operator of these names; their semantics are fixed as
compositions of reference primitives so that results can be compared with the reference:

* distances: nearest of the 27 periodic images under the cell metric, first minimum wins
  (PeriodicGeometryAdapter.forward, src/matterformer/geometry/adapters.py:176-190);
* attention: softmax(q.k * D^-1/2 + mask) v with a 0/-inf mask, the call
  RotaryMultiheadAttention.forward makes (src/matterformer/models/regular_attention.py:251-268);
  radius mask = distance <= cutoff (self included), local mask = band i-w/2 <= j <= i+w/2-1.

All compute runs in the C-ABI library; torch provides device memory and streams only.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from .simplicial import _DTYPE_CODE, _stream


def lattice_latent_to_cell(lattice: torch.Tensor) -> torch.Tensor:
    """Lower-triangular cell (rows = lattice vectors) from the "y1" latent
    ``[log a, log b, log c, cos alpha, cos beta, cos gamma]``.

    ref: lattice_latent_to_lower_triangular, src/matterformer/geometry/lattice.py:12-47
    (same clamps: log lengths to +-5, cosines to +-0.9999).
    """
    if lattice.ndim != 2 or lattice.shape[-1] != 6:
        raise ValueError(f"lattice must have shape (B, 6), got {tuple(lattice.shape)}")
    lat = lattice.float()
    lengths = lat[:, :3].clamp(-5.0, 5.0).exp()
    ca, cb, cg = lat[:, 3:].clamp(-0.9999, 0.9999).unbind(-1)
    sg = (1.0 - cg.square()).clamp_min(1e-8).sqrt()
    cell = lat.new_zeros(lat.shape[0], 3, 3)
    cell[:, 0, 0] = lengths[:, 0]
    cell[:, 1, 0] = lengths[:, 1] * cg
    cell[:, 1, 1] = lengths[:, 1] * sg
    cell[:, 2, 0] = lengths[:, 2] * cb
    cell[:, 2, 1] = lengths[:, 2] * (ca - cb * cg) / sg
    cell[:, 2, 2] = (lengths[:, 2].square() - cell[:, 2, 0].square() - cell[:, 2, 1].square()).sqrt().clamp_min(1e-8)
    return cell


def _as_cell(lattice_or_cell: torch.Tensor) -> torch.Tensor:
    if lattice_or_cell.ndim == 3 and lattice_or_cell.shape[-2:] == (3, 3):
        return lattice_or_cell.float().contiguous()
    return lattice_latent_to_cell(lattice_or_cell).contiguous()


def cell_grid_dims(cell: torch.Tensor, cutoff: float, max_per_axis: int = 64) -> torch.Tensor:
    """Cells per axis = floor(perpendicular width / cutoff), clamped to [1, max_per_axis]. (B,3) int32."""
    c = cell.double()
    a, b, cc = c[:, 0], c[:, 1], c[:, 2]
    vol = (a * torch.linalg.cross(b, cc)).sum(-1).abs()
    widths = torch.stack(
        [
            vol / torch.linalg.cross(b, cc).norm(dim=-1).clamp_min(1e-12),
            vol / torch.linalg.cross(cc, a).norm(dim=-1).clamp_min(1e-12),
            vol / torch.linalg.cross(a, b).norm(dim=-1).clamp_min(1e-12),
        ],
        dim=-1,
    )
    dims = torch.floor(widths / max(float(cutoff), 1e-12)).clamp(1, max_per_axis)
    return dims.to(torch.int32).contiguous()


def _num_atoms(num_atoms: Optional[torch.Tensor], batch: int, n: int, device) -> torch.Tensor:
    if num_atoms is None:
        return torch.full((batch,), n, device=device, dtype=torch.int32)
    return num_atoms.to(device=device, dtype=torch.int32).contiguous()


def knn_search_grid(cell: torch.Tensor, num_atoms: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Bins per axis (B,3) int32 and distance bounds (B,2) fp32 for the cell-list search (one small kernel).

    The bin edge is about 1.25x the radius of a sphere that holds k atoms at the structure's mean density, so the
    27 bins around an atom usually contain its k nearest neighbours; at most 16 bins per axis.
    """
    B = cell.shape[0]
    gd = torch.empty((B, 3), device=cell.device, dtype=torch.int32)
    bounds = torch.empty((B, 2), device=cell.device, dtype=torch.float32)
    n_max = 2**31 - 1
    with torch.cuda.device(cell.device):
        _lib.check(_lib.lib().mf_knn_search_grid(cell.data_ptr(), num_atoms.data_ptr(), B, n_max, int(k), gd.data_ptr(),
                                                 bounds.data_ptr(), _stream(cell.device)))  # fmt: skip
    return gd, bounds


def knn_topk(pos: torch.Tensor, lattice: torch.Tensor, num_atoms: Optional[torch.Tensor] = None, k: int = 16,
             include_self: bool = False, method: str = "cells") -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
    """k nearest periodic neighbours of every atom.

    ``pos`` (B,N,3) fractional fp32; ``lattice`` (B,6) latent or (B,3,3) cell; ``num_atoms`` (B).
    Returns ``idx`` int32 (B,N,k) and ``dist2`` fp32 (B,N,k) sorted by (distance, index); ties go to
    the lower index; missing neighbours are -1 / inf.  ``method`` is "cells" (cell list) or "pairs"
    (all pairs); both give the same bits.
    """
    if pos.device.type != "cuda":
        raise RuntimeError("knn_topk requires CUDA tensors")
    if pos.ndim != 3 or pos.shape[-1] != 3:
        raise ValueError(f"pos must have shape (B, N, 3), got {tuple(pos.shape)}")
    if method not in ("cells", "pairs"):
        raise ValueError(f"method must be 'cells' or 'pairs', got {method!r}")
    B, N, _ = pos.shape
    frac = pos.float().contiguous()
    cell = _as_cell(lattice).to(pos.device)
    na = _num_atoms(num_atoms, B, N, pos.device)
    idx = torch.empty((B, N, k), device=pos.device, dtype=torch.int32)
    d2 = torch.empty((B, N, k), device=pos.device, dtype=torch.float32)
    L = _lib.lib()
    with torch.cuda.device(pos.device):
        if method == "pairs":
            _lib.check(L.mf_knn_topk(frac.data_ptr(), cell.data_ptr(), na.data_ptr(), B, N, int(k),
                                     int(bool(include_self)), idx.data_ptr(), d2.data_ptr(), _stream(pos.device)))  # fmt: skip
        else:
            gd, bounds = knn_search_grid(cell, na, int(k))
            need = L.mf_knn_cells_workspace_bytes(B, N)
            ws = torch.empty(max(need, 1), device=pos.device, dtype=torch.uint8)
            _lib.check(L.mf_knn_topk_cells(frac.data_ptr(), cell.data_ptr(), na.data_ptr(), gd.data_ptr(),
                                           bounds.data_ptr(), B, N, int(k), int(bool(include_self)), idx.data_ptr(),
                                           d2.data_ptr(), ws.data_ptr(), need, _stream(pos.device)))  # fmt: skip
    return idx, d2


@dataclass
class RadiusBlocks:
    """Cell-sorted order and block list of one batch of structures (see mf_cell_sort_blocklist)."""

    perm: torch.Tensor  # (B,N) int32: original index of the s-th sorted atom
    block_count: torch.Tensor  # (B,T) int32
    block_cols: torch.Tensor  # (B,T,T) int32, ascending, -1 padded
    block_mask: torch.Tensor  # (B,T,T,32) int32 bit patterns (uint32 on the device side)
    num_atoms: torch.Tensor  # (B) int32
    cutoff: float
    tile: int = 32

    @property
    def inverse_perm(self) -> torch.Tensor:
        inv = torch.empty_like(self.perm)
        ar = torch.arange(self.perm.shape[1], device=self.perm.device, dtype=self.perm.dtype)
        inv.scatter_(1, self.perm.long(), ar.expand_as(self.perm))
        return inv


def build_radius_blocks(pos: torch.Tensor, lattice: torch.Tensor, num_atoms: Optional[torch.Tensor], cutoff: float,
                        tile: int = 32, grid_dims: Optional[torch.Tensor] = None) -> RadiusBlocks:  # fmt: skip
    """Cell-sort the atoms and list the 32x32 tiles that contain at least one pair within ``cutoff``."""
    if tile != 32:
        raise ValueError("only 32-atom tiles are supported")
    if pos.device.type != "cuda":
        raise RuntimeError("build_radius_blocks requires CUDA tensors")
    B, N, _ = pos.shape
    T = (N + 31) // 32
    dev = pos.device
    frac = pos.float().contiguous()
    cell = _as_cell(lattice).to(dev)
    na = _num_atoms(num_atoms, B, N, dev)
    gd = (cell_grid_dims(cell, cutoff) if grid_dims is None else grid_dims.to(device=dev, dtype=torch.int32)).contiguous()
    perm = torch.empty((B, N), device=dev, dtype=torch.int32)
    count = torch.empty((B, T), device=dev, dtype=torch.int32)
    cols = torch.empty((B, T, T), device=dev, dtype=torch.int32)
    mask = torch.empty((B, T, T, 32), device=dev, dtype=torch.int32)
    L = _lib.lib()
    need = L.mf_radius_blocks_workspace_bytes(B, N)
    ws = torch.empty(max(need, 1), device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        _lib.check(L.mf_cell_sort_blocklist(frac.data_ptr(), cell.data_ptr(), na.data_ptr(), gd.data_ptr(), B, N,
                                            float(cutoff), perm.data_ptr(), count.data_ptr(), cols.data_ptr(),
                                            mask.data_ptr(), ws.data_ptr(), need, _stream(dev)))  # fmt: skip
    return RadiusBlocks(perm=perm, block_count=count, block_cols=cols, block_mask=mask, num_atoms=na,
                        cutoff=float(cutoff))  # fmt: skip


_SPARSE_BACKEND = os.environ.get("MF_SPARSE_BACKEND", "auto")  # see set_sparse_backend


def set_sparse_backend(name: str) -> str:
    """Kernel family of the bf16 radius / local-window attention calls: ``"auto"`` (128-row tcgen05 tiles for radius
    lists over at least 256 tokens, 32-row warp-level tiles otherwise), ``"mma"`` or ``"tcgen05"``.  Returns the
    previous setting."""
    global _SPARSE_BACKEND
    if name not in _lib.MF_SPARSE_BACKEND:
        raise ValueError(f"unknown sparse attention backend {name!r}")
    prev, _SPARSE_BACKEND = _SPARSE_BACKEND, name
    return prev


def sparse_device_status(device=None) -> int:
    """Status word of the tcgen05 sparse-attention kernels on the current stream (0, or the code of an expired
    device-side wait).  Synchronises the stream."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    out = ctypes.c_int32(0)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().mf_sparse_attn_status(ctypes.byref(out), _stream(dev)))
    return int(out.value)


def _sparse_args(q, k, v, num_atoms, window, scale):
    B, H, N, D = q.shape
    a = _lib.MfSparseAttnArgs()
    a.backend = _lib.MF_SPARSE_BACKEND[_SPARSE_BACKEND] if q.dtype == torch.bfloat16 else 0
    a.batch, a.heads, a.tokens, a.head_dim = B, H, N, D
    a.dtype = _DTYPE_CODE[q.dtype]
    a.window = int(window)
    a.scale = float(scale)
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.num_atoms = num_atoms.data_ptr()
    return a


def _check_qkv(name, q, k, v):
    if q.device.type != "cuda":
        raise RuntimeError(f"{name} requires CUDA tensors")
    if q.dtype not in _DTYPE_CODE:
        raise RuntimeError(f"{name} only supports float16/bfloat16/float32 inputs, got {q.dtype}")
    if q.ndim != 4 or k.shape != q.shape or v.shape != q.shape:
        raise ValueError(f"{name}: q, k, v must share the shape (B, H, N, D)")
    if q.shape[-1] not in (32, 64, 128):
        raise ValueError(f"{name}: head_dim must be 32, 64 or 128, got {q.shape[-1]}")


class _SparseAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, num_atoms, kind, window, scale, block_count, block_cols, block_mask):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        B, H, N, D = q.shape
        out = torch.empty_like(q)
        lse = torch.empty((B, H, N), device=q.device, dtype=torch.float32)
        a = _sparse_args(q, k, v, num_atoms, window, scale)
        a.out, a.lse = out.data_ptr(), lse.data_ptr()
        L = _lib.lib()
        if kind == "radius":
            a.block_count, a.block_cols, a.block_mask = block_count.data_ptr(), block_cols.data_ptr(), block_mask.data_ptr()
            fn = L.mf_radius_attn_fwd
        else:
            fn = L.mf_local_attn_fwd
        with torch.cuda.device(q.device):
            _lib.check(fn(ctypes.byref(a), _stream(q.device)))
        ctx.kind, ctx.window, ctx.scale = kind, window, scale
        ctx.save_for_backward(q, k, v, out, lse, num_atoms, block_count, block_cols, block_mask)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        q, k, v, out, lse, num_atoms, block_count, block_cols, block_mask = ctx.saved_tensors
        grad_out = grad_out.to(q.dtype).contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
        a = _sparse_args(q, k, v, num_atoms, ctx.window, ctx.scale)
        a.out, a.lse, a.grad_out = out.data_ptr(), lse.data_ptr(), grad_out.data_ptr()
        a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        L = _lib.lib()
        need = L.mf_sparse_attn_bwd_workspace_bytes(ctypes.byref(a))
        ws = torch.empty(max(need, 1), device=q.device, dtype=torch.uint8)
        a.workspace, a.workspace_bytes = ws.data_ptr(), need
        if ctx.kind == "radius":
            a.block_count, a.block_cols, a.block_mask = block_count.data_ptr(), block_cols.data_ptr(), block_mask.data_ptr()
            fn = L.mf_radius_attn_bwd
        else:
            fn = L.mf_local_attn_bwd
        with torch.cuda.device(q.device):
            _lib.check(fn(ctypes.byref(a), _stream(q.device)))
        return dq, dk, dv, None, None, None, None, None, None, None


def radius_block_sparse_attention(q, k, v, blocks: RadiusBlocks, *, scale: Optional[float] = None,
                                  sorted_inputs: bool = True) -> torch.Tensor:  # fmt: skip
    """Attention over the pairs within ``blocks.cutoff``.

    ``q, k, v`` are (B,H,N,D).  With ``sorted_inputs`` the token axis is already in the cell-sorted
    order of ``blocks.perm``; otherwise tokens are gathered into that order and the result is
    scattered back.  Rows of padded atoms (and atoms without any neighbour) return zeros.
    """
    _check_qkv("radius_block_sparse_attention", q, k, v)
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    if not sorted_inputs:
        idx = blocks.perm.long()[:, None, :, None].expand_as(q)
        q, k, v = (torch.gather(t, 2, idx) for t in (q, k, v))
    out = _SparseAttention.apply(q, k, v, blocks.num_atoms, "radius", 0, scale, blocks.block_count,
                                 blocks.block_cols, blocks.block_mask)  # fmt: skip
    if not sorted_inputs:
        inv = blocks.inverse_perm.long()[:, None, :, None].expand_as(out)
        out = torch.gather(out, 2, inv)
    return out


def local_window_attention(q, k, v, num_atoms: Optional[torch.Tensor] = None, window: int = 64, *,
                           scale: Optional[float] = None) -> torch.Tensor:  # fmt: skip
    """Band attention over the token order: query i sees keys ``i - window/2 .. i + window/2 - 1``."""
    _check_qkv("local_window_attention", q, k, v)
    if window < 2 or window % 2:
        raise ValueError(f"window must be a positive even number, got {window}")
    B, H, N, D = q.shape
    na = _num_atoms(num_atoms, B, N, q.device)
    scale = D**-0.5 if scale is None else float(scale)
    empty = torch.empty(0, device=q.device, dtype=torch.int32)
    return _SparseAttention.apply(q, k, v, na, "local", int(window), scale, empty, empty, empty)


class _LocalAttentionPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, num_atoms, heads, window, scale):
        qkv = qkv.contiguous()
        B, N, W = qkv.shape
        D = W // (3 * heads)
        out = torch.empty((B, N, heads * D), device=qkv.device, dtype=qkv.dtype)
        lse = torch.empty((B, heads, N), device=qkv.device, dtype=torch.float32)
        a = _lib.MfLocalAttnPackedArgs(batch=B, heads=heads, tokens=N, head_dim=D, window=int(window), scale=float(scale),
                                       qkv=qkv.data_ptr(), num_atoms=num_atoms.data_ptr(), out=out.data_ptr(),
                                       lse=lse.data_ptr())  # fmt: skip
        with torch.cuda.device(qkv.device):
            _lib.check(_lib.lib().mf_local_attn_packed_fwd(ctypes.byref(a), _stream(qkv.device)))
        ctx.meta = (heads, int(window), float(scale))
        ctx.save_for_backward(qkv, out, lse, num_atoms)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        qkv, out, lse, num_atoms = ctx.saved_tensors
        heads, window, scale = ctx.meta
        B, N, W = qkv.shape
        D = W // (3 * heads)
        grad_out = grad_out.to(qkv.dtype).contiguous()
        grad_qkv = torch.empty_like(qkv)
        a = _lib.MfLocalAttnPackedArgs(batch=B, heads=heads, tokens=N, head_dim=D, window=window, scale=scale,
                                       qkv=qkv.data_ptr(), num_atoms=num_atoms.data_ptr(), out=out.data_ptr(),
                                       lse=lse.data_ptr(), grad_out=grad_out.data_ptr(),
                                       grad_qkv=grad_qkv.data_ptr())  # fmt: skip
        L = _lib.lib()
        need = int(L.mf_local_attn_packed_bwd_workspace_bytes(ctypes.byref(a)))
        ws = torch.empty(max(need, 16), device=qkv.device, dtype=torch.uint8)
        a.workspace, a.workspace_bytes = ws.data_ptr(), need
        with torch.cuda.device(qkv.device):
            _lib.check(L.mf_local_attn_packed_bwd(ctypes.byref(a), _stream(qkv.device)))
        return grad_qkv, None, None, None, None


def local_window_attention_packed(qkv: torch.Tensor, heads: int, num_atoms: Optional[torch.Tensor] = None,
                                  window: int = 64, *, scale: Optional[float] = None) -> torch.Tensor:  # fmt: skip
    """:func:`local_window_attention` on the packed projection of an attention layer: ``qkv`` (B, N, 3*H*D) bf16 as the
    input GEMM of ``nn.MultiheadAttention`` leaves it, result (B, N, H*D) as its output projection takes it; the
    gradient comes back in ``qkv``'s shape.  No head split before the core and no merge after it."""
    if qkv.device.type != "cuda" or qkv.dtype != torch.bfloat16 or qkv.ndim != 3 or qkv.shape[2] % (3 * heads):
        raise ValueError("local_window_attention_packed takes a CUDA bf16 (B, N, 3*H*D) tensor")
    D = qkv.shape[2] // (3 * heads)
    if D not in (32, 64, 128):
        raise ValueError(f"local_window_attention_packed: head_dim must be 32, 64 or 128, got {D}")
    if window < 2 or window % 2:
        raise ValueError(f"window must be a positive even number, got {window}")
    na = _num_atoms(num_atoms, qkv.shape[0], qkv.shape[1], qkv.device)
    return _LocalAttentionPacked.apply(qkv, na, int(heads), int(window), D**-0.5 if scale is None else float(scale))
