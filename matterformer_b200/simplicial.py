"""Host-side mirror of the reference's 2-simplicial attention kernel interface.

The two functions and the autograd ``Function`` here have the names-apart signatures, argument
meaning, return tuples and error behaviour of the reference's Triton backend
(src/matterformer/models/triton_simplicial_attention.py:790-926 and :929-1204, wrapped by
``_TritonTwoSimplicialAttentionFunction``, src/matterformer/models/simplicial_attention.py:347-637),
but run the sm_100a CUDA kernels through the C-ABI library.  :func:`install` rebinds the
reference module's kernel entry points to these functions, so existing ``impl="triton"`` /
``impl="auto"`` models, scripts and checkpoints run on this backend unchanged.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _lib

SUPPORTED_SIMPLICIAL_PRECISIONS = ("bf16_tc", "tf32", "ieee_fp32")

_DTYPE_CODE = {torch.float32: _lib.MF_DTYPE_F32, torch.bfloat16: _lib.MF_DTYPE_BF16, torch.float16: _lib.MF_DTYPE_F16}

# Backend used by the kernels: "auto" (tensor cores when the problem qualifies), "generic", "tcgen05".
_BACKEND = "auto"


def set_backend(name: str) -> str:
    """Select which kernel family serves simplicial calls; returns the previous setting."""
    global _BACKEND
    if name not in _lib.MF_BACKEND:
        raise ValueError(f"backend must be one of {tuple(_lib.MF_BACKEND)}, got {name!r}")
    prev, _BACKEND = _BACKEND, name
    return prev


def normalize_simplicial_precision(precision: str) -> str:
    """ref: normalize_simplicial_precision, triton_simplicial_attention.py:19-25."""
    normalized = str(precision).lower()
    if normalized not in SUPPORTED_SIMPLICIAL_PRECISIONS:
        raise ValueError(
            f"Unsupported simplicial_precision: {precision}. Expected one of {SUPPORTED_SIMPLICIAL_PRECISIONS}."
        )
    return normalized


# The status word of the most recent tensor-core call: a 4-byte copy of its own, so that no workspace (hundreds of
# megabytes after a backward pass) is kept alive just to read four bytes later.
_LAST_STATUS: Optional[torch.Tensor] = None
_CHECK_STATUS = os.environ.get("MF_CHECK_STATUS", "0") not in ("", "0")


def set_check_status(on: bool) -> bool:
    """When on, every tensor-core simplicial call reads its status word back (this synchronises the stream) and
    raises ``RuntimeError`` if a bounded device-side wait expired.  Skipped while a CUDA graph is being captured.
    Also switched on by the environment variable ``MF_CHECK_STATUS=1``.  Returns the previous setting."""
    global _CHECK_STATUS
    prev, _CHECK_STATUS = _CHECK_STATUS, bool(on)
    return prev


def _remember_status(ws: Optional[torch.Tensor]) -> None:
    global _LAST_STATUS
    if ws is None or ws.numel() < 4:
        return
    _LAST_STATUS = ws[:4].view(torch.int32).clone()
    if _CHECK_STATUS and not torch.cuda.is_current_stream_capturing():
        code = int(_LAST_STATUS.item())
        if code != 0:
            raise RuntimeError(f"a device-side wait of the tensor-core simplicial kernel expired (status {code}); "
                               "the outputs of this call are zeros")  # fmt: skip


def device_status() -> int:
    """Status word the most recent tensor-core simplicial kernel left in its workspace.

    0 means every bounded device-side wait completed; ``MF_ERR_DEVICE_TIMEOUT`` means a wait
    expired, the kernel gave up cleanly and the affected outputs are zeros (the backward pass then
    writes every gradient as zeros).  Reading it synchronises.
    """
    if _LAST_STATUS is None:
        return 0
    return int(_LAST_STATUS.item())


def _stream(device: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _check_inputs(name: str, q, k1, v1, k2, v2):
    if q.device.type != "cuda":
        raise RuntimeError(f"{name} requires CUDA tensors")
    if q.dtype not in _DTYPE_CODE:
        raise RuntimeError(f"the CUDA backend only supports float16/bfloat16/float32 inputs, got {q.dtype}")
    for t_name, t in (("k1", k1), ("v1", v1), ("k2", k2), ("v2", v2)):
        if t.shape != q.shape or t.dtype != q.dtype or t.device != q.device:
            raise ValueError(f"{t_name} must match q in shape, dtype and device")
    if q.ndim != 4:
        raise ValueError(f"q must have shape (B, H, N, D), got {tuple(q.shape)}")


def _mask_bytes(mask: torch.Tensor, shape, name: str) -> torch.Tensor:
    if tuple(mask.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(mask.shape)}")
    if mask.dtype != torch.bool:
        mask = mask != 0
    return mask.contiguous().view(torch.uint8)


MAX_RESIDUAL_RANK = 32


def _residual_group(kind: str, tensors: dict, shapes: dict):
    """fp32 contiguous copies of one low-rank residual group, or None when it is absent.

    ref: the has_low_rank_angle / has_low_rank_message tests of triton_simplicial_attention.py:839-871.
    """
    given = [t is not None for t in tensors.values()]
    if not any(given):
        return None
    if not all(given):
        raise ValueError(f"{', '.join(tensors)} must be given together")
    for name, t in tensors.items():
        want = shapes[name]
        if tuple(t.shape[: len(want)]) != tuple(want) or t.ndim != len(want) + (0 if name.endswith("gate") else 1):
            raise ValueError(f"{name} must have shape {tuple(want)}{'' if name.endswith('gate') else ' + (rank,)'}, "
                             f"got {tuple(t.shape)}")  # fmt: skip
    first = next(iter(tensors.values()))
    rank = int(first.shape[-1])
    if rank < 1 or rank > MAX_RESIDUAL_RANK:
        raise RuntimeError(f"the CUDA simplicial backend takes {kind} ranks up to {MAX_RESIDUAL_RANK}, got {rank}")
    return tuple(t.to(torch.float32).contiguous() for t in tensors.values()), rank


def _angle_group(left, right, gate, B, H, N):
    return _residual_group("angle", {"angle_left": left, "angle_right": right, "angle_gate": gate},
                           {"angle_left": (B, H, N, N), "angle_right": (B, H, N, N), "angle_gate": (B, H, N)})  # fmt: skip


def _message_group(left, right, basis, B, H, N, D):
    got = _residual_group("message", {"message_left": left, "message_right": right},
                          {"message_left": (B, H, N, N), "message_right": (B, H, N, N)})  # fmt: skip
    if got is None:
        if basis is not None:
            raise ValueError("message_basis given without message_left / message_right")
        return None
    (ml, mr), rank = got
    if basis is None or tuple(basis.shape) != (H, rank, D):
        raise ValueError(f"message_basis must have shape {(H, rank, D)}")
    return (ml, mr, basis.to(torch.float32).contiguous()), rank


def _factorized_bias(u, v_bias, w, gate, B, H, N):
    """fp32 contiguous copies of the factorized bias, or None when it is absent.

    ref: the has_bias test and the .contiguous().view(B*H, ...) reshapes of
    triton_simplicial_attention.py:829-837.
    """
    given = [t is not None for t in (u, v_bias, w, gate)]
    if not any(given):
        return None
    if not all(given):
        raise ValueError("u, v_bias, w and gate must be given together")
    for name, t in (("u", u), ("v_bias", v_bias), ("w", w)):
        if tuple(t.shape) != (B, H, N, N):
            raise ValueError(f"{name} must have shape {(B, H, N, N)}, got {tuple(t.shape)}")
    if tuple(gate.shape) != (B, H, N):
        raise ValueError(f"gate must have shape {(B, H, N)}, got {tuple(gate.shape)}")
    return tuple(t.to(torch.float32).contiguous() for t in (u, v_bias, w, gate))


def cuda_simplicial_attention_forward(
    q: torch.Tensor,
    k1: torch.Tensor,
    v1: torch.Tensor,
    k2: torch.Tensor,
    v2: torch.Tensor,
    *,
    query_valid: torch.Tensor,
    pair_key_valid: torch.Tensor,
    pair_valid: Optional[torch.Tensor],
    u: Optional[torch.Tensor] = None,
    v_bias: Optional[torch.Tensor] = None,
    w: Optional[torch.Tensor] = None,
    gate: Optional[torch.Tensor] = None,
    angle_left: Optional[torch.Tensor] = None,
    angle_right: Optional[torch.Tensor] = None,
    angle_gate: Optional[torch.Tensor] = None,
    message_left: Optional[torch.Tensor] = None,
    message_right: Optional[torch.Tensor] = None,
    message_basis: Optional[torch.Tensor] = None,
    precision: str = "bf16_tc",
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Forward pass. Returns ``(out[q.dtype], lse[fp32 (B,H,N)], out_fp32 (B,H,N,D))``.

    ref: triton_simplicial_attention_forward, triton_simplicial_attention.py:790-926.
    """
    _check_inputs("cuda_simplicial_attention_forward", q, k1, v1, k2, v2)
    precision = normalize_simplicial_precision(precision)
    B, H, N, D = q.shape
    q, k1, v1, k2, v2 = (t.contiguous() for t in (q, k1, v1, k2, v2))
    qv = _mask_bytes(query_valid, (B, N), "query_valid")
    kv = _mask_bytes(pair_key_valid, (B, N), "pair_key_valid")
    pv = _mask_bytes(pair_valid, (B, N, N), "pair_valid") if pair_valid is not None else None
    bias = _factorized_bias(u, v_bias, w, gate, B, H, N)
    angle = _angle_group(angle_left, angle_right, angle_gate, B, H, N)
    message = _message_group(message_left, message_right, message_basis, B, H, N, D)

    out32 = torch.empty((B, H, N, D), device=q.device, dtype=torch.float32)
    lse = torch.empty((B, H, N), device=q.device, dtype=torch.float32)
    out = out32 if q.dtype == torch.float32 else torch.empty_like(q)

    a = _lib.MfSimplicialFwdArgs()
    a.batch, a.heads, a.tokens, a.head_dim = B, H, N, D
    a.dtype = _DTYPE_CODE[q.dtype]
    a.precision = _lib.MF_PRECISION[precision]
    a.backend = _lib.MF_BACKEND[_BACKEND]
    a.q, a.k1, a.v1, a.k2, a.v2 = (t.data_ptr() for t in (q, k1, v1, k2, v2))
    a.query_valid, a.pair_key_valid = qv.data_ptr(), kv.data_ptr()
    a.pair_valid = pv.data_ptr() if pv is not None else None
    a.out, a.lse = out32.data_ptr(), lse.data_ptr()
    a.out_cast = out.data_ptr() if out is not out32 else None
    if bias is not None:
        a.u, a.v_bias, a.w, a.gate = (t.data_ptr() for t in bias)
    if angle is not None:
        a.angle_left, a.angle_right, a.angle_gate = (t.data_ptr() for t in angle[0])
        a.angle_rank = angle[1]
    if message is not None:
        a.message_left, a.message_right, a.message_basis = (t.data_ptr() for t in message[0])
        a.message_rank = message[1]
    L = _lib.lib()
    need = L.mf_simplicial_fwd_workspace_bytes(ctypes.byref(a))
    ws = torch.empty(max(need, 1), device=q.device, dtype=torch.uint8) if need else None
    a.workspace = ws.data_ptr() if ws is not None else None
    a.workspace_bytes = need
    with torch.cuda.device(q.device):
        _lib.check(L.mf_simplicial_fwd(ctypes.byref(a), _stream(q.device)))
    if L.mf_simplicial_fwd_backend(ctypes.byref(a)) == _lib.MF_BACKEND["tcgen05"]:
        _remember_status(ws)  # only the tensor-core kernels keep a status word there
    return out, lse, out32


def cuda_simplicial_attention_backward(
    grad_out: torch.Tensor,
    q: torch.Tensor,
    k1: torch.Tensor,
    v1: torch.Tensor,
    k2: torch.Tensor,
    v2: torch.Tensor,
    out: torch.Tensor,
    lse: torch.Tensor,
    *,
    query_valid: torch.Tensor,
    pair_key_valid: torch.Tensor,
    pair_valid: Optional[torch.Tensor],
    u: Optional[torch.Tensor] = None,
    v_bias: Optional[torch.Tensor] = None,
    w: Optional[torch.Tensor] = None,
    gate: Optional[torch.Tensor] = None,
    angle_left: Optional[torch.Tensor] = None,
    angle_right: Optional[torch.Tensor] = None,
    angle_gate: Optional[torch.Tensor] = None,
    message_left: Optional[torch.Tensor] = None,
    message_right: Optional[torch.Tensor] = None,
    message_basis: Optional[torch.Tensor] = None,
    precision: str = "bf16_tc",
    need_du: bool = False,
    need_dv_bias: bool = False,
    need_dw: bool = False,
    need_dgate: bool = False,
    need_dangle_left: bool = False,
    need_dangle_right: bool = False,
    need_dangle_gate: bool = False,
    need_dmessage_left: bool = False,
    need_dmessage_right: bool = False,
    need_dmessage_basis: bool = False,
):
    """Backward pass. Returns the reference's 15-tuple
    ``(dq, dk1, dv1, dk2, dv2, du, dv_bias, dw, dgate, dangle_left, dangle_right, dangle_gate,
    dmessage_left, dmessage_right, dmessage_basis)`` with ``None`` in the ten bias slots.

    ref: triton_simplicial_attention_backward, triton_simplicial_attention.py:929-1204.
    ``out`` is the fp32 output saved by the forward pass, ``lse`` its log-sum-exp.
    """
    _check_inputs("cuda_simplicial_attention_backward", q, k1, v1, k2, v2)
    precision = normalize_simplicial_precision(precision)
    B, H, N, D = q.shape
    q, k1, v1, k2, v2 = (t.contiguous() for t in (q, k1, v1, k2, v2))
    grad_out = grad_out.to(q.dtype).contiguous()
    out = out.to(torch.float32).contiguous()
    lse = lse.to(torch.float32).contiguous()
    qv = _mask_bytes(query_valid, (B, N), "query_valid")
    kv = _mask_bytes(pair_key_valid, (B, N), "pair_key_valid")
    pv = _mask_bytes(pair_valid, (B, N, N), "pair_valid") if pair_valid is not None else None
    grads = [torch.empty_like(q) for _ in range(5)]
    bias = _factorized_bias(u, v_bias, w, gate, B, H, N)
    bias_grads = [None, None, None, None]
    if bias is not None:
        for slot, (need_it, like) in enumerate(zip((need_du, need_dv_bias, need_dw, need_dgate), bias)):
            if need_it:
                bias_grads[slot] = torch.zeros_like(like)

    angle = _angle_group(angle_left, angle_right, angle_gate, B, H, N)
    message = _message_group(message_left, message_right, message_basis, B, H, N, D)
    angle_grads = [None, None, None]
    message_grads = [None, None, None]  # left, right, coefficients (the basis gradient is formed from them below)
    if angle is not None:
        for slot, (need_it, like) in enumerate(zip((need_dangle_left, need_dangle_right, need_dangle_gate), angle[0])):
            if need_it:
                angle_grads[slot] = torch.zeros_like(like)
    if message is not None:
        ml32, mr32, _ = message[0]
        if need_dmessage_left:
            message_grads[0] = torch.zeros_like(ml32)
        if need_dmessage_right:
            message_grads[1] = torch.zeros_like(mr32)
        if need_dmessage_basis:
            message_grads[2] = torch.zeros((B, H, N, message[1]), device=q.device, dtype=torch.float32)

    a = _lib.MfSimplicialBwdArgs()
    a.batch, a.heads, a.tokens, a.head_dim = B, H, N, D
    a.dtype = _DTYPE_CODE[q.dtype]
    a.precision = _lib.MF_PRECISION[precision]
    a.backend = _lib.MF_BACKEND[_BACKEND]
    a.grad_out = grad_out.data_ptr()
    a.q, a.k1, a.v1, a.k2, a.v2 = (t.data_ptr() for t in (q, k1, v1, k2, v2))
    a.out, a.lse = out.data_ptr(), lse.data_ptr()
    a.query_valid, a.pair_key_valid = qv.data_ptr(), kv.data_ptr()
    a.pair_valid = pv.data_ptr() if pv is not None else None
    a.dq, a.dk1, a.dv1, a.dk2, a.dv2 = (g.data_ptr() for g in grads)
    if bias is not None:
        a.u, a.v_bias, a.w, a.gate = (t.data_ptr() for t in bias)
        a.du, a.dv_bias, a.dw, a.dgate = (g.data_ptr() if g is not None else None for g in bias_grads)
    if angle is not None:
        a.angle_left, a.angle_right, a.angle_gate = (t.data_ptr() for t in angle[0])
        a.angle_rank = angle[1]
        a.dangle_left, a.dangle_right, a.dangle_gate = (g.data_ptr() if g is not None else None for g in angle_grads)
    if message is not None:
        a.message_left, a.message_right, a.message_basis = (t.data_ptr() for t in message[0])
        a.message_rank = message[1]
        a.dmessage_left, a.dmessage_right, a.message_coeff = (
            g.data_ptr() if g is not None else None for g in message_grads
        )
    L = _lib.lib()
    need = L.mf_simplicial_bwd_workspace_bytes(ctypes.byref(a))
    ws = torch.empty(max(need, 1), device=q.device, dtype=torch.uint8)
    a.workspace = ws.data_ptr()
    a.workspace_bytes = need
    with torch.cuda.device(q.device):
        _lib.check(L.mf_simplicial_bwd(ctypes.byref(a), _stream(q.device)))
    if L.mf_simplicial_bwd_backend(ctypes.byref(a)) == _lib.MF_BACKEND["tcgen05"]:
        _remember_status(ws)  # only the tensor-core kernels keep a status word there
    if bias is not None:  # the reference returns each bias gradient in the dtype of its operand (:1155-1160)
        bias_grads = [g.to(t.dtype) if g is not None else None for g, t in zip(bias_grads, (u, v_bias, w, gate))]
    if angle is not None:
        angle_grads = [g.to(t.dtype) if g is not None else None
                       for g, t in zip(angle_grads, (angle_left, angle_right, angle_gate))]  # fmt: skip
    if message is not None:
        if message_grads[2] is not None:  # d basis[h,r,:] = sum_{b,i} coeff[b,h,i,r] grad_out[b,h,i,:]
            message_grads[2] = torch.einsum("bhir,bhid->hrd", message_grads[2], grad_out.float()).to(message_basis.dtype)
        message_grads[0] = message_grads[0].to(message_left.dtype) if message_grads[0] is not None else None
        message_grads[1] = message_grads[1].to(message_right.dtype) if message_grads[1] is not None else None
    return (*grads, *bias_grads, *angle_grads, *message_grads)


class CudaTwoSimplicialAttentionFunction(torch.autograd.Function):
    """Autograd boundary with the reference's 21 positional arguments.

    ref: _TritonTwoSimplicialAttentionFunction, simplicial_attention.py:347-637.  Absent optionals
    arrive as 0-element tensors (:846-871); the kernel entry points are looked up in this module's
    globals at call time so that tests can replace them, as the reference's tests do (:755-756).
    """

    @staticmethod
    def forward(ctx, q, k1, v1, k2, v2, query_valid, pair_key_valid, pair_valid, u, v, w, gate, angle_left,
                angle_right, angle_gate, message_left, message_right, message_basis, precision_mode, chunk_size,
                debug_torch_backward):  # fmt: skip
        has_pair_valid = pair_valid.numel() > 0
        has_bias = u.numel() > 0
        has_angle = angle_left.numel() > 0
        has_message = message_left.numel() > 0
        out, lse, out_for_backward = cuda_simplicial_attention_forward(
            q, k1, v1, k2, v2,
            query_valid=query_valid,
            pair_key_valid=pair_key_valid,
            pair_valid=pair_valid if has_pair_valid else None,
            u=u if has_bias else None,
            v_bias=v if has_bias else None,
            w=w if has_bias else None,
            gate=gate if has_bias else None,
            angle_left=angle_left if has_angle else None,
            angle_right=angle_right if has_angle else None,
            angle_gate=angle_gate if has_angle else None,
            message_left=message_left if has_message else None,
            message_right=message_right if has_message else None,
            message_basis=message_basis if has_message else None,
            precision=precision_mode,
        )  # fmt: skip
        ctx.precision_mode = str(precision_mode)
        ctx.has_pair_valid = has_pair_valid
        ctx.has_bias, ctx.has_angle, ctx.has_message = has_bias, has_angle, has_message
        ctx.save_for_backward(q, k1, v1, k2, v2, query_valid, pair_key_valid, pair_valid, out_for_backward, lse,
                              u, v, w, gate, angle_left, angle_right, angle_gate, message_left, message_right,
                              message_basis)  # fmt: skip
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (q, k1, v1, k2, v2, query_valid, pair_key_valid, pair_valid, out, lse, u, v, w, gate, angle_left, angle_right,
         angle_gate, message_left, message_right, message_basis) = ctx.saved_tensors  # fmt: skip
        hb, ha, hm = ctx.has_bias, ctx.has_angle, ctx.has_message
        grads = cuda_simplicial_attention_backward(
            grad_out, q, k1, v1, k2, v2, out, lse,
            query_valid=query_valid,
            pair_key_valid=pair_key_valid,
            pair_valid=pair_valid if ctx.has_pair_valid else None,
            u=u if hb else None,
            v_bias=v if hb else None,
            w=w if hb else None,
            gate=gate if hb else None,
            precision=ctx.precision_mode,
            need_du=hb and ctx.needs_input_grad[8],
            need_dv_bias=hb and ctx.needs_input_grad[9],
            need_dw=hb and ctx.needs_input_grad[10],
            need_dgate=hb and ctx.needs_input_grad[11],
            angle_left=angle_left if ha else None,
            angle_right=angle_right if ha else None,
            angle_gate=angle_gate if ha else None,
            message_left=message_left if hm else None,
            message_right=message_right if hm else None,
            message_basis=message_basis if hm else None,
            need_dangle_left=ha and ctx.needs_input_grad[12],
            need_dangle_right=ha and ctx.needs_input_grad[13],
            need_dangle_gate=ha and ctx.needs_input_grad[14],
            need_dmessage_left=hm and ctx.needs_input_grad[15],
            need_dmessage_right=hm and ctx.needs_input_grad[16],
            need_dmessage_basis=hm and ctx.needs_input_grad[17],
        )  # fmt: skip
        dq, dk1, dv1, dk2, dv2 = grads[:5]
        return (dq, dk1, dv1, dk2, dv2, None, None, None, *grads[5:15], None, None, None)



def packed_projection_applies(proj: torch.Tensor, heads: int, head_dim: int) -> bool:
    """Whether :func:`simplicial_attention_packed` serves this projection: CUDA bf16 (B, N, 5*H*64) with at most 32
    tokens and a multiple of four heads (the kernels that pack four heads into one tile)."""
    return (proj.is_cuda and proj.dtype == torch.bfloat16 and proj.ndim == 3 and head_dim == 64 and heads % 4 == 0
            and proj.shape[1] <= 32 and proj.shape[2] == 5 * heads * head_dim and _BACKEND in ("auto", "tcgen05_tiles"))  # fmt: skip


class _PackedSimplicialAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, proj, query_valid, pair_key_valid, pair_valid, heads, q_scale):
        proj = proj.contiguous()
        B, N, W = proj.shape
        D = W // (5 * heads)
        qv = _mask_bytes(query_valid, (B, N), "query_valid")
        kv = _mask_bytes(pair_key_valid, (B, N), "pair_key_valid")
        pv = _mask_bytes(pair_valid, (B, N, N), "pair_valid") if pair_valid is not None else None
        out = torch.empty((B, N, heads * D), device=proj.device, dtype=proj.dtype)
        out32 = torch.empty((B, heads, N, D), device=proj.device, dtype=torch.float32)
        lse = torch.empty((B, heads, N), device=proj.device, dtype=torch.float32)
        a = _lib.MfSimplicialPackedArgs(batch=B, heads=heads, tokens=N, head_dim=D, q_scale=float(q_scale),
                                        proj=proj.data_ptr(), query_valid=qv.data_ptr(), pair_key_valid=kv.data_ptr(),
                                        pair_valid=pv.data_ptr() if pv is not None else None, out32=out32.data_ptr(),
                                        lse=lse.data_ptr(), out=out.data_ptr())  # fmt: skip
        L = _lib.lib()
        need = int(L.mf_simplicial_packed_fwd_workspace_bytes(ctypes.byref(a)))
        ws = torch.empty(max(need, 16), device=proj.device, dtype=torch.uint8)
        a.workspace, a.workspace_bytes = ws.data_ptr(), need
        with torch.cuda.device(proj.device):
            _lib.check(L.mf_simplicial_packed_fwd(ctypes.byref(a), _stream(proj.device)))
        _remember_status(ws)
        ctx.save_for_backward(proj, qv, kv, pv, out32, lse)
        ctx.meta = (heads, float(q_scale))
        return out

    @staticmethod
    def backward(ctx, grad_out):
        proj, qv, kv, pv, out32, lse = ctx.saved_tensors
        heads, q_scale = ctx.meta
        B, N, W = proj.shape
        D = W // (5 * heads)
        grad_out = grad_out.to(proj.dtype).contiguous()
        grad_proj = torch.empty_like(proj)
        a = _lib.MfSimplicialPackedArgs(batch=B, heads=heads, tokens=N, head_dim=D, q_scale=q_scale,
                                        proj=proj.data_ptr(), query_valid=qv.data_ptr(), pair_key_valid=kv.data_ptr(),
                                        pair_valid=pv.data_ptr() if pv is not None else None, out32=out32.data_ptr(),
                                        lse=lse.data_ptr(), grad_out=grad_out.data_ptr(),
                                        grad_proj=grad_proj.data_ptr())  # fmt: skip
        L = _lib.lib()
        need = int(L.mf_simplicial_packed_bwd_workspace_bytes(ctypes.byref(a)))
        ws = torch.empty(max(need, 16), device=proj.device, dtype=torch.uint8)
        a.workspace, a.workspace_bytes = ws.data_ptr(), need
        with torch.cuda.device(proj.device):
            _lib.check(L.mf_simplicial_packed_bwd(ctypes.byref(a), _stream(proj.device)))
        _remember_status(ws)
        return grad_proj, None, None, None, None, None


def simplicial_attention_packed(proj: torch.Tensor, *, heads: int, query_valid: torch.Tensor,
                                pair_key_valid: torch.Tensor, pair_valid: Optional[torch.Tensor] = None,
                                q_scale: Optional[float] = None) -> torch.Tensor:  # fmt: skip
    """2-simplicial attention straight on the layer's input projection.

    ``proj`` (B, N, 5*H*64) bf16 is the output of ``SimplicialAttention.in_proj`` (q, k1, v1, k2, v2 side by side, as
    ``_project_inputs`` chunks it, src/matterformer/models/simplicial_attention.py:718-725); the result (B, N, H*64) is
    what ``out_proj`` consumes (:965).  Neither the five head-major copies nor the permutation back exist; the
    gradient comes back as one tensor of ``proj``'s shape.  ``q_scale`` defaults to 64**-0.5."""
    if q_scale is None:
        q_scale = 0.125
    return _PackedSimplicialAttention.apply(proj, query_valid, pair_key_valid, pair_valid, int(heads), float(q_scale))


def simplicial_attention_cuda(q, k1, v1, k2, v2, *, query_valid, pair_key_valid, pair_valid=None,
                              factorized_bias=None, angle_residual=None, message_residual=None,
                              precision: str = "bf16_tc") -> torch.Tensor:  # fmt: skip
    """Differentiable 2-simplicial attention on projected heads ``(B,H,N,D)``; ``q`` pre-scaled.

    ``factorized_bias`` is an optional ``(u, v, w, gate)`` tuple: logits get ``gate_i (u_ij + v_ik + w_jk)``;
    ``angle_residual`` an optional ``(left, right, gate)`` tuple and ``message_residual`` an optional
    ``(left, right, basis)`` tuple of the low-rank residuals (simplicial_attention.py:50-104).
    """
    empty_f = q.new_empty(0)
    empty_b = torch.empty(0, device=q.device, dtype=torch.bool)
    u, v, w, gate = factorized_bias if factorized_bias is not None else (empty_f,) * 4
    al, ar, ag = angle_residual if angle_residual is not None else (empty_f,) * 3
    ml, mr, mb = message_residual if message_residual is not None else (empty_f,) * 3
    return CudaTwoSimplicialAttentionFunction.apply(
        q.contiguous(), k1.contiguous(), v1.contiguous(), k2.contiguous(), v2.contiguous(),
        query_valid.contiguous(), pair_key_valid.contiguous(),
        pair_valid.contiguous() if pair_valid is not None else empty_b,
        u, v, w, gate, al, ar, ag, ml, mr, mb,
        precision, 128, False,
    )  # fmt: skip


def install(reference_module=None) -> None:
    """Rebind the reference's kernel entry points to this backend.

    ``_TritonTwoSimplicialAttentionFunction`` resolves ``triton_simplicial_attention_forward`` /
    ``_backward`` and ``TRITON_AVAILABLE`` from the globals of
    ``matterformer.models.simplicial_attention`` at call time (simplicial_attention.py:377,581,746),
    which is also how the reference's own tests swap kernels.  After this call every reference
    ``SimplicialAttention(impl="triton"|"auto")`` runs the sm_100a kernels, the factorized bias and
    the low-rank angle / message residuals (ranks up to 32) included.
    """
    if reference_module is None:
        import matterformer.models.simplicial_attention as reference_module  # type: ignore
    _lib.lib()  # fail now if the library is missing

    saved = getattr(reference_module, "_matterformer_b200_saved", None)
    original_reason = saved[3] if saved is not None else reference_module.SimplicialAttention._triton_unavailable_reason

    def _reason(self, *, x, factorized_bias, angle_residual, message_residual, message_basis, logit_bias_fn,
                return_attn):  # fmt: skip
        reason = original_reason(self, x=x, factorized_bias=factorized_bias, angle_residual=angle_residual,
                                 message_residual=message_residual, message_basis=message_basis,
                                 logit_bias_fn=logit_bias_fn, return_attn=return_attn)  # fmt: skip
        if reason is None:
            for res in (angle_residual, message_residual):
                if res is not None and int(res.left.shape[-1]) > MAX_RESIDUAL_RANK:
                    return f"the CUDA backend takes residual ranks up to {MAX_RESIDUAL_RANK}"
        return reason

    if not hasattr(reference_module, "_matterformer_b200_saved"):
        reference_module._matterformer_b200_saved = (
            reference_module.TRITON_AVAILABLE,
            getattr(reference_module, "triton_simplicial_attention_forward", None),
            getattr(reference_module, "triton_simplicial_attention_backward", None),
            original_reason,
        )
    reference_module.TRITON_AVAILABLE = True
    reference_module.triton_simplicial_attention_forward = cuda_simplicial_attention_forward
    reference_module.triton_simplicial_attention_backward = cuda_simplicial_attention_backward
    reference_module.SimplicialAttention._triton_unavailable_reason = _reason


def uninstall(reference_module=None) -> None:
    """Undo :func:`install`: the reference module gets its own kernel entry points back."""
    if reference_module is None:
        import matterformer.models.simplicial_attention as reference_module  # type: ignore
    saved = getattr(reference_module, "_matterformer_b200_saved", None)
    if saved is None:
        return
    available, fwd, bwd, reason = saved
    reference_module.TRITON_AVAILABLE = available
    reference_module.triton_simplicial_attention_forward = fwd
    reference_module.triton_simplicial_attention_backward = bwd
    reference_module.SimplicialAttention._triton_unavailable_reason = reason
    del reference_module._matterformer_b200_saved
