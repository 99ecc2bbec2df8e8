"""ctypes binding of the C-ABI library declared in ``include/matterformer_b200.h``.

The library is the only compute backend of this package: there is no Python or CPU fallback.
:func:`lib` raises if the shared object is missing, so a GPU box that lost the built ``.so``
fails loudly instead of silently computing somewhere else.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int32, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libmatterformer_b200.so"

MF_OK = 0
MF_ERR_INVALID_ARGUMENT = -1
MF_ERR_UNSUPPORTED = -2
MF_ERR_WORKSPACE_TOO_SMALL = -3
MF_ERR_CUDA = -4
MF_ERR_DEVICE_TIMEOUT = -5

MF_DTYPE_F32, MF_DTYPE_BF16, MF_DTYPE_F16 = 0, 1, 2
MF_PRECISION = {"bf16_tc": 0, "tf32": 1, "ieee_fp32": 2}
MF_BACKEND = {"auto": 0, "generic": 1, "tcgen05": 2, "tcgen05_tiles": 3}
MF_SPARSE_BACKEND = {"auto": 0, "mma": 1, "tcgen05": 2}

# Every symbol include/matterformer_b200.h declares.
EXPORTED_SYMBOLS = (
    "mf_simplicial_fwd_backend",
    "mf_simplicial_bwd_backend",
    "mf_simplicial_row_plan",
    "mf_simplicial_fwd_workspace_bytes",
    "mf_simplicial_bwd_workspace_bytes",
    "mf_simplicial_fwd",
    "mf_simplicial_bwd",
    "mf_simplicial_fwd_noalloc",
    "mf_simplicial_noalloc_status",
    "mf_selftest_wait_timeout",
    "mf_knn_topk",
    "mf_knn_search_grid",
    "mf_knn_cells_workspace_bytes",
    "mf_knn_topk_cells",
    "mf_radius_blocks_workspace_bytes",
    "mf_cell_sort_blocklist",
    "mf_sparse_attn_bwd_workspace_bytes",
    "mf_radius_attn_fwd",
    "mf_radius_attn_bwd",
    "mf_local_attn_fwd",
    "mf_local_attn_bwd",
    "mf_sparse_attn_status",
    "mf_local_attn_packed_bwd_workspace_bytes",
    "mf_local_attn_packed_fwd",
    "mf_local_attn_packed_bwd",
    "mf_last_error",
    "mf_version",
    "mf_feature_flags",
    "mf_ln_modulate_fwd",
    "mf_ln_modulate_bwd",
    "mf_gated_residual_fwd",
    "mf_gated_residual_bwd",
    "mf_column_sums_workspace_bytes",
    "mf_column_sums",
    "mf_gelu_tanh_fwd",
    "mf_gelu_tanh_bwd",
    "mf_split_heads",
    "mf_merge_heads",
    "mf_simplicial_packed_fwd_workspace_bytes",
    "mf_simplicial_packed_bwd_workspace_bytes",
    "mf_simplicial_packed_fwd",
    "mf_simplicial_packed_bwd",
    "mf_pair_head_bwd_workspace_bytes",
    "mf_pair_head_fwd",
    "mf_pair_head_bwd",
    "mf_profile_enable",
    "mf_profile_read",
)


class MfSimplicialFwdArgs(Structure):
    _fields_ = [
        ("batch", c_int32),
        ("heads", c_int32),
        ("tokens", c_int32),
        ("head_dim", c_int32),
        ("dtype", c_int32),
        ("precision", c_int32),
        ("backend", c_int32),
        ("reserved0", c_int32),
        ("q", c_void_p),
        ("k1", c_void_p),
        ("v1", c_void_p),
        ("k2", c_void_p),
        ("v2", c_void_p),
        ("query_valid", c_void_p),
        ("pair_key_valid", c_void_p),
        ("pair_valid", c_void_p),
        ("u", c_void_p),
        ("v_bias", c_void_p),
        ("w", c_void_p),
        ("gate", c_void_p),
        ("angle_left", c_void_p),
        ("angle_right", c_void_p),
        ("angle_gate", c_void_p),
        ("message_left", c_void_p),
        ("message_right", c_void_p),
        ("message_basis", c_void_p),
        ("angle_rank", c_int32),
        ("message_rank", c_int32),
        ("out", c_void_p),
        ("lse", c_void_p),
        ("out_cast", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
    ]


class MfSimplicialBwdArgs(Structure):
    _fields_ = [
        ("batch", c_int32),
        ("heads", c_int32),
        ("tokens", c_int32),
        ("head_dim", c_int32),
        ("dtype", c_int32),
        ("precision", c_int32),
        ("backend", c_int32),
        ("reserved0", c_int32),
        ("grad_out", c_void_p),
        ("q", c_void_p),
        ("k1", c_void_p),
        ("v1", c_void_p),
        ("k2", c_void_p),
        ("v2", c_void_p),
        ("out", c_void_p),
        ("lse", c_void_p),
        ("query_valid", c_void_p),
        ("pair_key_valid", c_void_p),
        ("pair_valid", c_void_p),
        ("dq", c_void_p),
        ("dk1", c_void_p),
        ("dv1", c_void_p),
        ("dk2", c_void_p),
        ("dv2", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
        ("u", c_void_p),
        ("v_bias", c_void_p),
        ("w", c_void_p),
        ("gate", c_void_p),
        ("du", c_void_p),
        ("dv_bias", c_void_p),
        ("dw", c_void_p),
        ("dgate", c_void_p),
        ("angle_left", c_void_p),
        ("angle_right", c_void_p),
        ("angle_gate", c_void_p),
        ("message_left", c_void_p),
        ("message_right", c_void_p),
        ("message_basis", c_void_p),
        ("angle_rank", c_int32),
        ("message_rank", c_int32),
        ("dangle_left", c_void_p),
        ("dangle_right", c_void_p),
        ("dangle_gate", c_void_p),
        ("dmessage_left", c_void_p),
        ("dmessage_right", c_void_p),
        ("message_coeff", c_void_p),
    ]


class MfSparseAttnArgs(Structure):
    _fields_ = [
        ("batch", c_int32),
        ("heads", c_int32),
        ("tokens", c_int32),
        ("head_dim", c_int32),
        ("dtype", c_int32),
        ("window", c_int32),
        ("scale", c_float),
        ("backend", c_int32),
        ("q", c_void_p),
        ("k", c_void_p),
        ("v", c_void_p),
        ("num_atoms", c_void_p),
        ("block_count", c_void_p),
        ("block_cols", c_void_p),
        ("block_mask", c_void_p),
        ("out", c_void_p),
        ("lse", c_void_p),
        ("grad_out", c_void_p),
        ("dq", c_void_p),
        ("dk", c_void_p),
        ("dv", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
    ]


class MfLocalAttnPackedArgs(Structure):
    _fields_ = [
        ("batch", c_int32),
        ("heads", c_int32),
        ("tokens", c_int32),
        ("head_dim", c_int32),
        ("window", c_int32),
        ("scale", c_float),
        ("qkv", c_void_p),
        ("num_atoms", c_void_p),
        ("out", c_void_p),
        ("lse", c_void_p),
        ("grad_out", c_void_p),
        ("grad_qkv", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
    ]


class MfSimplicialPackedArgs(Structure):
    _fields_ = [
        ("batch", c_int32),
        ("heads", c_int32),
        ("tokens", c_int32),
        ("head_dim", c_int32),
        ("q_scale", c_float),
        ("reserved0", c_int32),
        ("proj", c_void_p),
        ("query_valid", c_void_p),
        ("pair_key_valid", c_void_p),
        ("pair_valid", c_void_p),
        ("out32", c_void_p),
        ("lse", c_void_p),
        ("out", c_void_p),
        ("grad_out", c_void_p),
        ("grad_proj", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
    ]


class MfPairHeadArgs(Structure):
    _fields_ = [
        ("batch", c_int32),
        ("tokens", c_int32),
        ("hidden", c_int32),
        ("n_rbf", c_int32),
        ("dtype", c_int32),
        ("gamma", c_float),
        ("a", c_void_p),
        ("b", c_void_p),
        ("coords", c_void_p),
        ("valid", c_void_p),
        ("w_rbf", c_void_p),
        ("w_out", c_void_p),
        ("b_out", c_void_p),
        ("centers", c_void_p),
        ("out", c_void_p),
        ("grad_out", c_void_p),
        ("grad_a", c_void_p),
        ("grad_b", c_void_p),
        ("grad_w_rbf", c_void_p),
        ("grad_w_out", c_void_p),
        ("grad_b_out", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
    ]


_LIB = None


def lib() -> ctypes.CDLL:
    """Load (once) and return the C-ABI library with argument types declared."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m matterformer_b200.build` "
            "(this package has no fallback implementation)"
        )
    L = ctypes.CDLL(str(LIB_PATH))
    L.mf_simplicial_fwd_workspace_bytes.argtypes = [POINTER(MfSimplicialFwdArgs)]
    L.mf_simplicial_fwd_workspace_bytes.restype = c_size_t
    L.mf_simplicial_bwd_workspace_bytes.argtypes = [POINTER(MfSimplicialBwdArgs)]
    L.mf_simplicial_bwd_workspace_bytes.restype = c_size_t
    L.mf_simplicial_row_plan.argtypes = [c_int32, c_int32, POINTER(c_int32 * 4)]
    L.mf_simplicial_row_plan.restype = c_int32
    L.mf_simplicial_fwd.argtypes = [POINTER(MfSimplicialFwdArgs), c_void_p]
    L.mf_simplicial_fwd.restype = c_int32
    L.mf_simplicial_bwd.argtypes = [POINTER(MfSimplicialBwdArgs), c_void_p]
    L.mf_simplicial_bwd.restype = c_int32
    L.mf_simplicial_fwd_noalloc.argtypes = [POINTER(MfSimplicialFwdArgs), c_void_p]
    L.mf_simplicial_fwd_noalloc.restype = c_int32
    L.mf_simplicial_noalloc_status.argtypes = [POINTER(c_int32), c_void_p]
    L.mf_simplicial_noalloc_status.restype = c_int32
    L.mf_selftest_wait_timeout.argtypes = [c_void_p, ctypes.c_int64, c_void_p]
    L.mf_selftest_wait_timeout.restype = c_int32
    L.mf_knn_topk.argtypes = [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p]
    L.mf_knn_topk.restype = c_int32
    L.mf_knn_search_grid.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p]
    L.mf_knn_search_grid.restype = c_int32
    L.mf_knn_cells_workspace_bytes.argtypes = [c_int32, c_int32]
    L.mf_knn_cells_workspace_bytes.restype = c_size_t
    L.mf_knn_topk_cells.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                    c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]  # fmt: skip
    L.mf_knn_topk_cells.restype = c_int32
    L.mf_radius_blocks_workspace_bytes.argtypes = [c_int32, c_int32]
    L.mf_radius_blocks_workspace_bytes.restype = c_size_t
    L.mf_cell_sort_blocklist.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_float,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p,
    ]  # fmt: skip
    L.mf_cell_sort_blocklist.restype = c_int32
    L.mf_sparse_attn_bwd_workspace_bytes.argtypes = [POINTER(MfSparseAttnArgs)]
    L.mf_sparse_attn_bwd_workspace_bytes.restype = c_size_t
    for name in ("mf_radius_attn_fwd", "mf_radius_attn_bwd", "mf_local_attn_fwd", "mf_local_attn_bwd"):
        fn = getattr(L, name)
        fn.argtypes = [POINTER(MfSparseAttnArgs), c_void_p]
        fn.restype = c_int32
    L.mf_last_error.argtypes = [c_char_p, c_size_t]
    L.mf_last_error.restype = c_size_t
    L.mf_version.argtypes = []
    L.mf_version.restype = c_int32
    L.mf_feature_flags.argtypes = []
    L.mf_feature_flags.restype = c_int32
    L.mf_ln_modulate_fwd.argtypes = [c_void_p, c_int32, c_void_p, c_void_p, c_int32, c_int32, c_int32, ctypes.c_float,
                                     c_int32, c_void_p, c_void_p, c_void_p, c_void_p]  # fmt: skip
    L.mf_ln_modulate_fwd.restype = c_int32
    L.mf_ln_modulate_bwd.argtypes = [c_void_p, c_int32, c_void_p, c_int32, c_void_p, c_void_p, c_void_p, c_int32,
                                     c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p]  # fmt: skip
    L.mf_ln_modulate_bwd.restype = c_int32
    L.mf_gated_residual_fwd.argtypes = [c_void_p, c_int32, c_void_p, c_void_p, c_int32, c_void_p, c_int32, c_int32,
                                        c_int32, c_void_p, c_void_p]  # fmt: skip
    L.mf_gated_residual_fwd.restype = c_int32
    L.mf_gated_residual_bwd.argtypes = [c_void_p, c_int32, c_void_p, c_void_p, c_int32, c_void_p, c_int32, c_int32,
                                        c_int32, c_void_p, c_void_p, c_void_p, c_void_p]  # fmt: skip
    L.mf_gated_residual_bwd.restype = c_int32
    L.mf_column_sums_workspace_bytes.argtypes = [ctypes.c_int64, c_int32]
    L.mf_column_sums_workspace_bytes.restype = c_size_t
    L.mf_column_sums.argtypes = [c_void_p, c_int32, ctypes.c_int64, c_int32, c_void_p, c_void_p, c_size_t, c_void_p]
    L.mf_column_sums.restype = c_int32
    L.mf_gelu_tanh_fwd.argtypes = [c_void_p, c_int32, ctypes.c_int64, c_void_p, c_void_p]
    L.mf_gelu_tanh_fwd.restype = c_int32
    L.mf_gelu_tanh_bwd.argtypes = [c_void_p, c_void_p, c_int32, ctypes.c_int64, c_int32, c_void_p, c_void_p, c_void_p,
                                   c_size_t, c_void_p]  # fmt: skip
    L.mf_gelu_tanh_bwd.restype = c_int32
    L.mf_split_heads.argtypes = [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                 c_void_p]  # fmt: skip
    L.mf_split_heads.restype = c_int32
    L.mf_merge_heads.argtypes = [c_void_p, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32,
                                 c_void_p]  # fmt: skip
    L.mf_merge_heads.restype = c_int32
    for fn in (L.mf_simplicial_packed_fwd_workspace_bytes, L.mf_simplicial_packed_bwd_workspace_bytes):
        fn.argtypes = [POINTER(MfSimplicialPackedArgs)]
        fn.restype = c_size_t
    for fn in (L.mf_simplicial_packed_fwd, L.mf_simplicial_packed_bwd):
        fn.argtypes = [POINTER(MfSimplicialPackedArgs), c_void_p]
        fn.restype = c_int32
    L.mf_local_attn_packed_bwd_workspace_bytes.argtypes = [POINTER(MfLocalAttnPackedArgs)]
    L.mf_local_attn_packed_bwd_workspace_bytes.restype = c_size_t
    for fn in (L.mf_local_attn_packed_fwd, L.mf_local_attn_packed_bwd):
        fn.argtypes = [POINTER(MfLocalAttnPackedArgs), c_void_p]
        fn.restype = c_int32
    L.mf_sparse_attn_status.argtypes = [POINTER(c_int32), c_void_p]
    L.mf_sparse_attn_status.restype = c_int32
    L.mf_pair_head_bwd_workspace_bytes.argtypes = [POINTER(MfPairHeadArgs)]
    L.mf_pair_head_bwd_workspace_bytes.restype = c_size_t
    for fn in (L.mf_pair_head_fwd, L.mf_pair_head_bwd):
        fn.argtypes = [POINTER(MfPairHeadArgs), c_void_p]
        fn.restype = c_int32
    L.mf_simplicial_fwd_backend.argtypes = [POINTER(MfSimplicialFwdArgs)]
    L.mf_simplicial_fwd_backend.restype = c_int32
    L.mf_simplicial_bwd_backend.argtypes = [POINTER(MfSimplicialBwdArgs)]
    L.mf_simplicial_bwd_backend.restype = c_int32
    L.mf_profile_enable.argtypes = [c_int32]
    L.mf_profile_enable.restype = c_int32
    L.mf_profile_read.argtypes = [c_int32, POINTER(ctypes.c_double), POINTER(c_int32)]
    L.mf_profile_read.restype = c_int32
    _LIB = L
    return L


def last_error() -> str:
    buf = ctypes.create_string_buffer(512)
    lib().mf_last_error(buf, 512)
    return buf.value.decode("utf-8", "replace")


def profile_enable(on: bool) -> None:
    check(lib().mf_profile_enable(int(bool(on))))


def profile_read(which: int) -> tuple[float, int]:
    """(summed device milliseconds, launches) of the main kernel `which` (0 forward, 1 backward)."""
    ms, n = ctypes.c_double(0.0), c_int32(0)
    check(lib().mf_profile_read(which, ctypes.byref(ms), ctypes.byref(n)))
    return ms.value, n.value


def check(rc: int) -> None:
    """Translate a C-ABI return code into the exception the reference's Python layer would raise."""
    if rc == MF_OK:
        return
    msg = last_error()
    if rc == MF_ERR_INVALID_ARGUMENT:
        raise ValueError(msg)
    raise RuntimeError(msg)


def simplicial_row_plan(n_queries: int, valid_keys: int) -> tuple[int, int, int, int]:
    """(query ranges, queries per range, first keys per step, steps per range) of the row-packed kernels."""
    out = (c_int32 * 4)()
    check(lib().mf_simplicial_row_plan(int(n_queries), int(valid_keys), ctypes.byref(out)))
    return tuple(int(v) for v in out)
