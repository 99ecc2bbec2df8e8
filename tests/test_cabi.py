"""The C-ABI library loads and exports every symbol the public header declares (no compute calls)."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

from matterformer_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def _declared_symbols():
    text = (ROOT / "include" / "matterformer_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mf_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    names = _declared_symbols()
    assert set(names) == set(_lib.EXPORTED_SYMBOLS)
    L = _lib.lib()
    for n in names:
        assert hasattr(L, n), f"{n} is declared in the header but not exported"
    assert L.mf_version() >= 100


def test_struct_layout_matches_header():
    # pointer/size fields are 8 bytes, ints 4: the struct sizes follow from the header's field lists
    assert ctypes.sizeof(_lib.MfSimplicialFwdArgs) == 8 * 4 + 18 * 8 + 2 * 4 + 5 * 8
    assert ctypes.sizeof(_lib.MfSimplicialBwdArgs) == 8 * 4 + 16 * 8 + 2 * 8 + 8 * 8 + 6 * 8 + 2 * 4 + 6 * 8
    assert ctypes.sizeof(_lib.MfSparseAttnArgs) == 8 * 4 + 13 * 8 + 2 * 8
    assert ctypes.sizeof(_lib.MfPairHeadArgs) == 6 * 4 + 16 * 8 + 8


def test_argument_errors_need_no_gpu():
    L = _lib.lib()
    assert L.mf_simplicial_fwd(None, None) == _lib.MF_ERR_INVALID_ARGUMENT
    assert "null argument struct" in _lib.last_error()
    a = _lib.MfSimplicialFwdArgs()
    a.batch, a.heads, a.tokens, a.head_dim = 1, 1, 4, 256
    assert L.mf_simplicial_fwd(ctypes.byref(a), None) == _lib.MF_ERR_INVALID_ARGUMENT
    assert "head_dim <= 128" in _lib.last_error()
    a.head_dim, a.dtype = 8, 7
    assert L.mf_simplicial_fwd(ctypes.byref(a), None) == _lib.MF_ERR_INVALID_ARGUMENT
    assert "only supports float16/bfloat16/float32" in _lib.last_error()
    assert L.mf_knn_topk(None, None, None, 1, 1, 4, 0, None, None, None) == _lib.MF_ERR_INVALID_ARGUMENT
    assert L.mf_knn_topk(None, None, None, 0, 1, 4, 0, None, None, None) == _lib.MF_OK  # empty batch: nothing to do
    s = _lib.MfSparseAttnArgs()
    s.head_dim = 48
    assert L.mf_local_attn_fwd(ctypes.byref(s), None) == _lib.MF_ERR_INVALID_ARGUMENT
    ph = _lib.MfPairHeadArgs(batch=1, tokens=4, hidden=64, n_rbf=16)
    assert L.mf_pair_head_fwd(ctypes.byref(ph), None) == _lib.MF_ERR_INVALID_ARGUMENT
    assert "hidden width of 128" in _lib.last_error()
    ph.hidden, ph.batch = 128, 0
    assert L.mf_pair_head_fwd(ctypes.byref(ph), None) == _lib.MF_OK  # empty batch: nothing to do
    assert L.mf_pair_head_bwd_workspace_bytes(ctypes.byref(ph)) == 0
    assert L.mf_column_sums(None, _lib.MF_DTYPE_BF16, 4, 12, None, None, 0, None) == _lib.MF_ERR_INVALID_ARGUMENT
    assert "multiple of 8" in _lib.last_error()
    assert L.mf_column_sums(16, _lib.MF_DTYPE_BF16, 4, 16, 16, None, 0, None) == _lib.MF_ERR_WORKSPACE_TOO_SMALL
    assert L.mf_column_sums(8, _lib.MF_DTYPE_BF16, 4, 16, 16, None, 0, None) == _lib.MF_ERR_INVALID_ARGUMENT  # unaligned
    assert L.mf_column_sums_workspace_bytes(29696, 2560) >= 2560 * 4
    with pytest.raises(ValueError):
        _lib.check(_lib.MF_ERR_INVALID_ARGUMENT)
    with pytest.raises(RuntimeError):
        _lib.check(_lib.MF_ERR_UNSUPPORTED)


def test_python_layer_rejects_cpu_tensors():
    import matterformer_b200 as mfb

    q = torch.zeros(1, 1, 4, 8)
    ok = torch.ones(1, 4, dtype=torch.bool)
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        mfb.cuda_simplicial_attention_forward(q, q, q, q, q, query_valid=ok, pair_key_valid=ok, pair_valid=None)
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        mfb.knn_topk(torch.zeros(1, 4, 3), torch.zeros(1, 6))
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        mfb.local_window_attention(q, q, q)
    with pytest.raises(ValueError, match="Unsupported simplicial_precision"):
        mfb.simplicial.normalize_simplicial_precision("fp8")


def test_row_plan_invariants():
    """The packing of (query, first key) pairs onto 128-row tiles, for every size the tensor-core kernels take."""
    assert _lib.simplicial_row_plan(0, 5) == (0, 0, 0, 0)
    assert _lib.simplicial_row_plan(5, 0) == (0, 0, 0, 0)
    for nq in range(1, 193):
        for nk in (1, 2, 7, 29, 64, 100, 128, 129, 150, 181, 192):
            tiles, rt, groups, steps = _lib.simplicial_row_plan(nq, nk)
            assert 1 <= tiles <= 8 and 1 <= groups <= 8
            assert rt * groups <= 128, "a step's rows fit the tile"
            assert tiles * rt >= nq and (tiles - 1) * rt < nq, "every query in exactly one non-empty range"
            assert (steps - 1) * groups < nk <= steps * groups, "every valid first key in exactly one step"
            # never worse than one query per row
            plain_tiles = -(-nq // 128)
            assert tiles * steps <= plain_tiles * nk


def test_unaligned_tensors_are_caught_before_any_launch():
    """Kernels use 16-byte vector accesses.  A tensor that starts off a 16-byte boundary is refused by the sparse and
    AdaLN entry points and sent to the element-wise kernel by the simplicial ones -- decided on the host, no GPU."""
    L = _lib.lib()
    ok, off = 0x7F0000001000, 0x7F0000001002  # fake device addresses: validation never dereferences them
    s = _lib.MfSparseAttnArgs()
    s.batch, s.heads, s.tokens, s.head_dim, s.dtype, s.window = 1, 1, 32, 64, _lib.MF_DTYPE_BF16, 64
    s.q, s.k, s.v, s.out, s.lse, s.num_atoms = off, ok, ok, ok, ok, ok
    assert L.mf_local_attn_fwd(ctypes.byref(s), None) == _lib.MF_ERR_INVALID_ARGUMENT
    assert "not 16-byte aligned" in _lib.last_error()
    assert L.mf_ln_modulate_fwd(off, _lib.MF_DTYPE_F32, ok, ok, 1, 4, 64, 1e-6, _lib.MF_DTYPE_F32, ok, ok, ok, None) \
        == _lib.MF_ERR_INVALID_ARGUMENT  # fmt: skip
    assert "not 16-byte aligned" in _lib.last_error()
    a = _lib.MfSimplicialFwdArgs()
    a.batch, a.heads, a.tokens, a.head_dim = 2, 2, 40, 64
    a.dtype, a.precision, a.backend = _lib.MF_DTYPE_BF16, _lib.MF_PRECISION["bf16_tc"], _lib.MF_BACKEND["auto"]
    a.q, a.k1, a.v1, a.k2, a.v2, a.out, a.lse = ok, ok, ok, ok, ok, ok, ok
    assert L.mf_simplicial_fwd_backend(ctypes.byref(a)) == _lib.MF_BACKEND["tcgen05"]
    a.k2 = off
    assert L.mf_simplicial_fwd_backend(ctypes.byref(a)) == _lib.MF_BACKEND["generic"]
    a.backend = _lib.MF_BACKEND["tcgen05"]  # asked for explicitly: a clear error instead of a misaligned access
    a.query_valid = a.pair_key_valid = ok
    assert L.mf_simplicial_fwd(ctypes.byref(a), None) == _lib.MF_ERR_UNSUPPORTED
    assert "16-byte boundaries" in _lib.last_error()
