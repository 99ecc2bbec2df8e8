"""ctypes front end of ``geom_oracle.c`` (TEST INFRASTRUCTURE, see that file's header).

Builds ``oracle/libmf_oracle.so`` with the Makefile beside it when missing.  All functions take and
return CPU torch tensors.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import c_float, c_int32, c_void_p
from pathlib import Path

import torch

_DIR = Path(__file__).resolve().parent
_SO = _DIR / "libmf_oracle.so"
_LIB = None


def build(force: bool = False) -> Path:
    src = _DIR / "geom_oracle.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_DIR), "-B", "libmf_oracle.so"], check=True, capture_output=True)
    return _SO


def _lib():
    global _LIB
    if _LIB is None:
        if not _SO.exists():
            build()
        L = ctypes.CDLL(str(_SO))
        L.mfo_set_threads.argtypes = [c_int32]
        L.mfo_get_threads.restype = c_int32
        L.mfo_pair_dist2.argtypes = [c_void_p, c_void_p, c_int32, c_void_p]
        L.mfo_knn_topk.argtypes = [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p]
        L.mfo_cell_sort_blocklist.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_float,
                                              c_void_p, c_void_p, c_void_p, c_void_p]  # fmt: skip
        _LIB = L
    return _LIB


def set_threads(n: int) -> None:
    _lib().mfo_set_threads(int(n))


def _f32(t):
    return t.detach().cpu().float().contiguous()


def _i32(t):
    return t.detach().cpu().to(torch.int32).contiguous()


def pair_dist2(frac: torch.Tensor, cell: torch.Tensor) -> torch.Tensor:
    """(N,N) minimum-image squared distances of one structure (fixed-order fp32 formula)."""
    frac, cell = _f32(frac), _f32(cell)
    n = frac.shape[0]
    out = torch.empty(n, n, dtype=torch.float32)
    _lib().mfo_pair_dist2(frac.data_ptr(), cell.data_ptr(), n, out.data_ptr())
    return out


def knn_topk(frac, cell, num_atoms, k: int, include_self: bool = False):
    frac, cell, na = _f32(frac), _f32(cell), _i32(num_atoms)
    B, N, _ = frac.shape
    idx = torch.empty(B, N, k, dtype=torch.int32)
    d2 = torch.empty(B, N, k, dtype=torch.float32)
    _lib().mfo_knn_topk(frac.data_ptr(), cell.data_ptr(), na.data_ptr(), B, N, k, int(include_self), idx.data_ptr(),
                        d2.data_ptr())  # fmt: skip
    return idx, d2


def cell_sort_blocklist(frac, cell, num_atoms, grid_dims, cutoff: float):
    frac, cell, na, gd = _f32(frac), _f32(cell), _i32(num_atoms), _i32(grid_dims)
    B, N, _ = frac.shape
    T = (N + 31) // 32
    perm = torch.empty(B, N, dtype=torch.int32)
    count = torch.empty(B, T, dtype=torch.int32)
    cols = torch.empty(B, T, T, dtype=torch.int32)
    mask = torch.empty(B, T, T, 32, dtype=torch.int32)
    _lib().mfo_cell_sort_blocklist(frac.data_ptr(), cell.data_ptr(), na.data_ptr(), gd.data_ptr(), B, N, float(cutoff),
                                   perm.data_ptr(), count.data_ptr(), cols.data_ptr(), mask.data_ptr())  # fmt: skip
    return perm, count, cols, mask


def default_threads() -> int:
    return os.cpu_count() or 1
