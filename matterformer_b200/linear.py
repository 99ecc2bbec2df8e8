"""Linear layers of the trunk under bf16 autocast without the per-call casts.

``torch.autocast`` casts every fp32 weight and bias to bf16 inside each ``F.linear`` call and casts every weight /
bias gradient back to fp32 afterwards: for the trunk of the reference (``AdaLNBlock``, models/transformer.py:228-316,
five Linear layers per block) that is some 600 small cast kernels per training step, a quarter of all launches once the
batch is split over eight GPUs.  Here each parameter keeps a bf16 copy that is refreshed for all layers at once at the
start of a forward pass (one multi-tensor copy), and the backward pass writes the weight gradient in fp32 straight out of
the GEMM and the bias gradient comes from this library's column-sum kernels (``mf_column_sums``: one read of the output
gradient, fixed order of additions).  The GEMMs themselves stay library calls (cuBLAS).
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch
import torch.nn.functional as F

from .fused import column_sums, column_sums_applies, gelu_tanh_applies, gelu_tanh_backward, gelu_tanh_forward

_SHADOW = "_mf_bf16_copy"  # attribute on the parameter: (bf16 tensor, parameter version it was made from)


def _bf16_autocast() -> bool:
    return torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16


def linear_bf16_applies(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """CUDA, an fp32 parameter, and bf16 arithmetic asked for (autocast or a bf16 input)."""
    return x.is_cuda and weight.is_cuda and weight.dtype == torch.float32 and (x.dtype == torch.bfloat16 or _bf16_autocast())


def _current(p: torch.Tensor) -> Optional[torch.Tensor]:
    entry = getattr(p, _SHADOW, None)
    if entry is None:
        return None
    copy, version = entry
    if version != p._version or copy.device != p.device or copy.shape != p.shape:
        return None
    return copy


def bf16_copy(p: torch.Tensor) -> torch.Tensor:
    """The parameter's bf16 copy, refreshed if the parameter changed since it was made."""
    copy = _current(p)
    if copy is None:
        entry = getattr(p, _SHADOW, None)
        copy = entry[0] if entry is not None and entry[0].device == p.device and entry[0].shape == p.shape else None
        with torch.no_grad():
            if copy is None:
                copy = p.detach().to(torch.bfloat16)
            else:
                copy.copy_(p.detach())
        setattr(p, _SHADOW, (copy, p._version))
    return copy


def refresh_bf16_copies(params: Iterable[torch.Tensor], *, force: bool = False) -> None:
    """Bring the bf16 copies of ``params`` up to date with one multi-tensor copy.  ``force`` copies even when the version
    counters say nothing changed: a step captured in a CUDA graph must contain the copy, because a replay updates the
    parameters without running this Python code again."""
    stale_dst, stale_src = [], []
    for p in params:
        if p is None or not p.is_cuda or p.dtype != torch.float32:
            continue
        entry = getattr(p, _SHADOW, None)
        if entry is None or entry[0].device != p.device or entry[0].shape != p.shape:
            bf16_copy(p)  # first use: allocates
            if not force:
                continue
            entry = getattr(p, _SHADOW)
        if force or entry[1] != p._version:
            stale_dst.append(entry[0])
            stale_src.append(p.detach())
            setattr(p, _SHADOW, (entry[0], p._version))
    if stale_dst:
        with torch.no_grad():
            torch._foreach_copy_(stale_dst, stale_src)


_MM_OUT_DTYPE = True  # torch.mm(..., out_dtype=) exists; cleared on the first refusal


def _mm_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a @ b for bf16 operands with the fp32 accumulator written out unrounded."""
    global _MM_OUT_DTYPE
    if _MM_OUT_DTYPE:
        try:
            return torch.mm(a, b, out_dtype=torch.float32)
        except (TypeError, RuntimeError):
            _MM_OUT_DTYPE = False
    return torch.mm(a, b).float()


class _LinearBf16(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        w16 = bf16_copy(weight)
        b16 = bf16_copy(bias) if bias is not None else None
        ctx.save_for_backward(x, w16)
        ctx.has_bias = bias is not None
        with torch.autocast("cuda", enabled=False):
            return F.linear(x, w16, b16)

    @staticmethod
    def backward(ctx, dy):
        x, w16 = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.dtype != torch.bfloat16:
            dy2 = dy2.to(torch.bfloat16)
        dx = dw = db = None
        with torch.autocast("cuda", enabled=False):
            if ctx.needs_input_grad[0]:
                dx = torch.mm(dy2, w16).view(x.shape)
            if ctx.needs_input_grad[1]:
                dw = _mm_f32(dy2.t(), x.reshape(-1, x.shape[-1]))
            if ctx.has_bias and ctx.needs_input_grad[2]:
                dyc = dy2 if dy2.is_contiguous() else dy2.contiguous()
                db = column_sums(dyc) if column_sums_applies(dyc) else dyc.sum(0, dtype=torch.float32)
        return dx, dw, db


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """``F.linear`` in bf16 on fp32 parameters (what autocast computes), returning bf16.  Falls back to ``F.linear``
    where :func:`linear_bf16_applies` says no.  A step that is captured into a CUDA graph and updates the parameters
    must call ``refresh_bf16_copies(params, force=True)`` inside the captured region before its first layer (the trunk
    does): the version counters this function checks do not advance during replays."""
    if not linear_bf16_applies(x, weight):
        return F.linear(x, weight, bias)
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    return _LinearBf16.apply(x, weight, bias)


class _LinearGeluBf16(torch.autograd.Function):
    """fc1 + GELU(tanh) of the block's MLP.  The backward pass forms the gradient of the pre-activation and the bias
    gradient in one sweep over (pre-activation, incoming gradient)."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        w16 = bf16_copy(weight)
        b16 = bf16_copy(bias) if bias is not None else None
        with torch.autocast("cuda", enabled=False):
            pre = F.linear(x, w16, b16)
        ctx.save_for_backward(x, w16, pre)
        ctx.has_bias = bias is not None
        return gelu_tanh_forward(pre)

    @staticmethod
    def backward(ctx, dact):
        x, w16, pre = ctx.saved_tensors
        cols = pre.shape[-1]
        dact2 = dact.reshape(-1, cols)
        if dact2.dtype != torch.bfloat16:
            dact2 = dact2.to(torch.bfloat16)
        dpre, sums = gelu_tanh_backward(pre.reshape(-1, cols), dact2.contiguous())
        dx = dw = None
        with torch.autocast("cuda", enabled=False):
            if ctx.needs_input_grad[0]:
                dx = torch.mm(dpre, w16).view(x.shape)
            if ctx.needs_input_grad[1]:
                dw = _mm_f32(dpre.t(), x.reshape(-1, x.shape[-1]))
        return dx, dw, (sums if ctx.has_bias and ctx.needs_input_grad[2] else None)


def linear_gelu_bf16(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """``gelu(F.linear(x, weight, bias), approximate="tanh")`` in bf16 on fp32 parameters; plain torch calls where
    :func:`linear_bf16_applies` says no."""
    if not (linear_bf16_applies(x, weight) and weight.shape[0] % 8 == 0):
        return F.gelu(F.linear(x, weight, bias), approximate="tanh")
    if x.dtype != torch.bfloat16:
        x = x.to(torch.bfloat16)
    return _LinearGeluBf16.apply(x.contiguous(), weight, bias)
