"""The allocation-free forward entry point against the regular one.

``mf_simplicial_fwd_noalloc`` serves callers that hold only their input and output buffers and may not
allocate device memory (code living inside another runtime's pool, loops that must keep off the allocator,
hosts whose allocator is frozen).  Its scratch is an array inside the library image.  This file is named so
that pytest collects it last: if it fails, every other test has already run.

The test drives the entry point directly through the C ABI -- it fills ``MfSimplicialFwdArgs`` by hand and
passes no workspace -- twice in a row with different batches, so the second call runs on whatever the first
one left in the shared scratch, and compares every output with ``mf_simplicial_fwd`` (same kernels, so the
results must be bit-identical).
"""
import ctypes

import pytest
import torch

from matterformer_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(B, H, N, seed, n_lo):
    g = torch.Generator().manual_seed(seed)
    t = [(torch.randn(B, H, N, 64, generator=g) / 8).bfloat16().to(DEV) for _ in range(5)]
    n = torch.randint(n_lo, N + 1, (B,), generator=g)
    valid = (torch.arange(N)[None, :] < n[:, None]).to(DEV)
    return t, valid


def _call(entry, t, valid, workspace):
    B, H, N, D = t[0].shape
    out32 = torch.full((B, H, N, D), float("nan"), device=DEV, dtype=torch.float32)
    lse = torch.full((B, H, N), float("nan"), device=DEV, dtype=torch.float32)
    out = torch.empty(B, H, N, D, device=DEV, dtype=torch.bfloat16)
    mask = valid.contiguous().view(torch.uint8)
    a = _lib.MfSimplicialFwdArgs()
    a.batch, a.heads, a.tokens, a.head_dim = B, H, N, D
    a.dtype, a.precision, a.backend = _lib.MF_DTYPE_BF16, _lib.MF_PRECISION["bf16_tc"], _lib.MF_BACKEND["auto"]
    a.q, a.k1, a.v1, a.k2, a.v2 = (x.data_ptr() for x in t)
    a.query_valid = a.pair_key_valid = mask.data_ptr()
    a.out, a.lse, a.out_cast = out32.data_ptr(), lse.data_ptr(), out.data_ptr()
    L = _lib.lib()
    if workspace:
        need = L.mf_simplicial_fwd_workspace_bytes(ctypes.byref(a))
        ws = torch.empty(need, device=DEV, dtype=torch.uint8)
        a.workspace, a.workspace_bytes = ws.data_ptr(), need
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(getattr(L, entry)(ctypes.byref(a), stream))
    torch.cuda.synchronize()
    return out32, lse, out


def test_noalloc_forward_matches_regular_entry_point_twice():
    for seed, (B, H, N, n_lo) in enumerate([(5, 4, 150, 90), (9, 2, 64, 3)]):
        t, valid = _inputs(B, H, N, seed, n_lo)
        ref = _call("mf_simplicial_fwd", t, valid, workspace=True)
        got = _call("mf_simplicial_fwd_noalloc", t, valid, workspace=False)
        for r, g_ in zip(ref, got):
            assert torch.equal(r, g_)  # identical kernels and inputs: identical bits
        assert torch.isfinite(got[0]).all()
        # the status word of the built-in scratch is readable without any allocation
        status = ctypes.c_int32(-99)
        _lib.check(_lib.lib().mf_simplicial_noalloc_status(ctypes.byref(status), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        torch.cuda.synchronize()
        assert status.value == 0


def test_noalloc_rejects_what_it_cannot_serve():
    L = _lib.lib()
    a = _lib.MfSimplicialFwdArgs()
    a.batch, a.heads, a.tokens, a.head_dim = 5000, 1, 8, 64
    a.dtype, a.precision = _lib.MF_DTYPE_BF16, _lib.MF_PRECISION["bf16_tc"]
    assert L.mf_simplicial_fwd_noalloc(ctypes.byref(a), None) == _lib.MF_ERR_INVALID_ARGUMENT
    assert "at most 4096" in _lib.last_error()
    a.batch, a.dtype = 2, _lib.MF_DTYPE_F32
    assert L.mf_simplicial_fwd_noalloc(ctypes.byref(a), None) == _lib.MF_ERR_UNSUPPORTED
