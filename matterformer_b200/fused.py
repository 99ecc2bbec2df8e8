"""Fused element-wise passes of the trunk's adaptive-LayerNorm block on the C-ABI kernels.

``ln_modulate(x, shift, scale)`` = ``LayerNorm(x) * (1 + scale[:, None]) + shift[:, None]`` and
``gated_residual(x, gate, a)`` = ``x + gate[:, None] * a`` (AdaLNBlock.forward of the reference,
src/matterformer/models/transformer.py:242-253, 308-316), each one pass over the (B, N, C) tensor forward
and one backward instead of a chain of element-wise kernels.  ``x`` is the residual stream, fp32 or bf16
(bf16 is what autocast leaves it in); ``shift``, ``scale`` and ``gate`` are used in fp32 and their gradients
come back in their own dtype.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib

_CODE = {torch.float32: _lib.MF_DTYPE_F32, torch.bfloat16: _lib.MF_DTYPE_BF16}
MAX_CHANNELS = 1024


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def fused_applies(x: torch.Tensor) -> bool:
    """The kernels take a CUDA fp32 / bf16 (B, N, C) residual stream; C a multiple of 8, at most ``MAX_CHANNELS``."""
    return x.is_cuda and x.dtype in _CODE and x.ndim == 3 and x.shape[-1] <= MAX_CHANNELS and x.shape[-1] % 8 == 0


class _LnModulate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shift, scale, eps, out_dtype):
        ctx.param_dtypes = (shift.dtype, scale.dtype)
        x, shift, scale = x.contiguous(), shift.float().contiguous(), scale.float().contiguous()
        B, N, C = x.shape
        h = torch.empty((B, N, C), device=x.device, dtype=out_dtype)
        mean = torch.empty((B, N), device=x.device, dtype=torch.float32)
        rstd = torch.empty_like(mean)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().mf_ln_modulate_fwd(x.data_ptr(), _CODE[x.dtype], shift.data_ptr(), scale.data_ptr(),
                                                     B, N, C, float(eps), _CODE[out_dtype], h.data_ptr(),
                                                     mean.data_ptr(), rstd.data_ptr(), _stream(x.device)))  # fmt: skip
        ctx.save_for_backward(x, scale, mean, rstd)
        return h

    @staticmethod
    def backward(ctx, dh):
        x, scale, mean, rstd = ctx.saved_tensors
        B, N, C = x.shape
        if dh.dtype not in _CODE:
            dh = dh.float()
        dh = dh.contiguous()
        dx = torch.empty_like(x)
        dshift = torch.empty((B, C), device=x.device, dtype=torch.float32)
        dscale = torch.empty_like(dshift)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().mf_ln_modulate_bwd(dh.data_ptr(), _CODE[dh.dtype], x.data_ptr(), _CODE[x.dtype],
                                                     scale.data_ptr(), mean.data_ptr(), rstd.data_ptr(), B, N, C,
                                                     dx.data_ptr(), dshift.data_ptr(), dscale.data_ptr(),
                                                     _stream(x.device)))  # fmt: skip
        return dx, dshift.to(ctx.param_dtypes[0]), dscale.to(ctx.param_dtypes[1]), None, None


class _GatedResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, a, pad):
        ctx.gate_dtype = gate.dtype
        x, gate = x.contiguous(), gate.float().contiguous()
        if a.dtype not in _CODE:
            a = a.float()
        a = a.contiguous()
        pad = pad.to(torch.uint8).contiguous() if pad is not None else None
        B, N, C = x.shape
        y = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().mf_gated_residual_fwd(x.data_ptr(), _CODE[x.dtype], gate.data_ptr(), a.data_ptr(),
                                                        _CODE[a.dtype], pad.data_ptr() if pad is not None else None,
                                                        B, N, C, y.data_ptr(), _stream(x.device)))  # fmt: skip
        ctx.save_for_backward(gate, a, pad)
        return y

    @staticmethod
    def backward(ctx, dy):
        gate, a, pad = ctx.saved_tensors
        B, N, C = a.shape
        if dy.dtype not in _CODE:
            dy = dy.float()
        dy = dy.contiguous()
        da = torch.empty_like(a)
        dx = torch.empty_like(dy) if pad is not None else None
        dgate = torch.empty((B, C), device=a.device, dtype=torch.float32)
        with torch.cuda.device(a.device):
            _lib.check(_lib.lib().mf_gated_residual_bwd(dy.data_ptr(), _CODE[dy.dtype], gate.data_ptr(), a.data_ptr(),
                                                        _CODE[a.dtype], pad.data_ptr() if pad is not None else None,
                                                        B, N, C, da.data_ptr(), dx.data_ptr() if dx is not None else None,
                                                        dgate.data_ptr(), _stream(a.device)))  # fmt: skip
        return (dy if dx is None else dx), dgate.to(ctx.gate_dtype), da, None


def ln_modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, *, eps: float,
                out_dtype: torch.dtype = torch.float32) -> torch.Tensor:  # fmt: skip
    """``LayerNorm(x) * (1 + scale[:, None, :]) + shift[:, None, :]`` in ``out_dtype`` (fp32 or bf16)."""
    return _LnModulate.apply(x, shift, scale, eps, out_dtype)


def gated_residual(x: torch.Tensor, gate: torch.Tensor, a: torch.Tensor,
                   pad_mask: Optional[torch.Tensor] = None) -> torch.Tensor:  # fmt: skip
    """``x + gate[:, None, :] * a`` in ``x``'s dtype; with ``pad_mask`` (B, N) bool, followed by
    ``.masked_fill(pad_mask[..., None], 0)`` in the same pass (forward and backward)."""
    return _GatedResidual.apply(x, gate, a, pad_mask)


class _SplitModulation(torch.autograd.Function):
    """(B, 6 C) -> six contiguous fp32 (B, C) tensors in one copy; the backward pass gathers the six gradients in one
    concatenation and one cast."""

    @staticmethod
    def forward(ctx, mod):
        B, W = mod.shape
        ctx.in_dtype = mod.dtype
        out = torch.empty((6, B, W // 6), device=mod.device, dtype=torch.float32)
        out.copy_(mod.view(B, 6, W // 6).transpose(0, 1))
        return tuple(out.unbind(0))

    @staticmethod
    def backward(ctx, *grads):
        g = torch.stack([t if t is not None else torch.zeros_like(grads[0]) for t in grads], dim=1)  # (B, 6, C) fp32
        return g.reshape(g.shape[0], -1).to(ctx.in_dtype)


def split_modulation(mod: torch.Tensor):
    """The six AdaLN modulation vectors ``shift_a, scale_a, gate_a, shift_m, scale_m, gate_m`` of
    ``self.ada_ln(cond).chunk(6, dim=-1)`` (transformer.py:242-244) as contiguous fp32 tensors, which is what the fused
    LayerNorm-modulate and gated-residual kernels read."""
    if mod.ndim != 2 or mod.shape[1] % 6 != 0 or not mod.is_cuda:
        return mod.chunk(6, dim=-1)
    return _SplitModulation.apply(mod)


def column_sums_applies(x: torch.Tensor) -> bool:
    return (x.is_cuda and x.ndim == 2 and x.dtype in _CODE and x.is_contiguous() and x.shape[1] % 8 == 0
            and x.shape[1] >= 8 and x.data_ptr() % 16 == 0)  # fmt: skip


def column_sums(x: torch.Tensor) -> torch.Tensor:
    """``x.sum(0)`` of a (rows, cols) fp32 / bf16 matrix in fp32, in a fixed order of additions: the bias gradient of a
    Linear layer from its output gradient.  No autograd (it is used inside backward passes)."""
    if not column_sums_applies(x):
        raise ValueError("column_sums needs a contiguous CUDA fp32 / bf16 matrix with a multiple of 8 columns")
    L = _lib.lib()
    rows, cols = x.shape
    out = torch.empty(cols, device=x.device, dtype=torch.float32)
    need = L.mf_column_sums_workspace_bytes(rows, cols)
    ws = torch.empty(max(need, 16), device=x.device, dtype=torch.uint8)
    with torch.cuda.device(x.device):
        _lib.check(L.mf_column_sums(x.data_ptr(), _CODE[x.dtype], rows, cols, out.data_ptr(), ws.data_ptr(), need,
                                    _stream(x.device)))  # fmt: skip
    return out


def gelu_tanh_applies(x: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype in _CODE and x.is_contiguous() and x.ndim >= 1 and x.shape[-1] % 8 == 0
            and x.data_ptr() % 16 == 0)  # fmt: skip


def gelu_tanh_forward(x: torch.Tensor) -> torch.Tensor:
    """``F.gelu(x, approximate="tanh")`` (no autograd; see :func:`matterformer_b200.linear.linear_gelu_bf16`)."""
    if not gelu_tanh_applies(x):
        raise ValueError("gelu_tanh_forward needs a contiguous CUDA fp32 / bf16 tensor with a multiple of 8 columns")
    y = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().mf_gelu_tanh_fwd(x.data_ptr(), _CODE[x.dtype], x.numel(), y.data_ptr(), _stream(x.device)))
    return y


def gelu_tanh_backward(pre: torch.Tensor, dy: torch.Tensor):
    """``(dy * gelu'(pre), column sums of that product in fp32)`` for (rows, cols) matrices: the gradient of the
    pre-activation and, in the same sweep, the bias gradient of the Linear layer that produced it."""
    if not (gelu_tanh_applies(pre) and gelu_tanh_applies(dy) and pre.ndim == 2 and pre.shape == dy.shape and pre.dtype == dy.dtype):
        raise ValueError("gelu_tanh_backward needs two contiguous CUDA matrices of one shape and type")
    L = _lib.lib()
    rows, cols = pre.shape
    dx = torch.empty_like(pre)
    sums = torch.empty(cols, device=pre.device, dtype=torch.float32)
    need = L.mf_column_sums_workspace_bytes(rows, cols)
    ws = torch.empty(max(need, 16), device=pre.device, dtype=torch.uint8)
    with torch.cuda.device(pre.device):
        _lib.check(L.mf_gelu_tanh_bwd(pre.data_ptr(), dy.data_ptr(), _CODE[pre.dtype], rows, cols, dx.data_ptr(),
                                      sums.data_ptr(), ws.data_ptr(), need, _stream(pre.device)))  # fmt: skip
    return dx, sums


def _ptr_array(tensors):
    arr = (ctypes.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr() if t is not None else None
    return arr


def _scale_array(scales, groups):
    if scales is None:
        return None
    arr = (ctypes.c_float * groups)()
    for i in range(groups):
        arr[i] = float(scales[i])
    return arr


def heads_layout_applies(packed: torch.Tensor, heads: int, groups: int) -> bool:
    """CUDA fp32 / bf16 (B, N, groups*heads*D) with head rows of a multiple of 16 bytes."""
    if not (packed.is_cuda and packed.dtype in _CODE and packed.ndim == 3 and 1 <= groups <= 8):
        return False
    width = packed.shape[-1]
    if width % (groups * heads):
        return False
    return ((width // (groups * heads)) * packed.element_size()) % 16 == 0


class _SplitHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, packed, groups, heads, scales):
        packed = packed.contiguous()
        B, N, W = packed.shape
        D = W // (groups * heads)
        outs = torch.empty((groups, B, heads, N, D), device=packed.device, dtype=packed.dtype)
        views = list(outs.unbind(0))
        with torch.cuda.device(packed.device):
            _lib.check(_lib.lib().mf_split_heads(packed.data_ptr(), _ptr_array(views), _scale_array(scales, groups),
                                                 groups, B, N, heads, D, _CODE[packed.dtype],
                                                 _stream(packed.device)))  # fmt: skip
        ctx.meta = (groups, heads, scales, B, N, D, packed.dtype)
        return tuple(views)

    @staticmethod
    def backward(ctx, *grads):
        groups, heads, scales, B, N, D, dtype = ctx.meta
        gs = [g.to(dtype).contiguous() if g is not None else None for g in grads]
        dev = next(g.device for g in gs if g is not None)
        packed = torch.empty((B, N, groups * heads * D), device=dev, dtype=dtype)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib().mf_merge_heads(_ptr_array(gs), _scale_array(scales, groups), packed.data_ptr(),
                                                 groups, B, N, heads, D, _CODE[dtype], _stream(dev)))  # fmt: skip
        return packed, None, None, None


class _MergeHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        B, H, N, D = x.shape
        packed = torch.empty((B, N, H * D), device=x.device, dtype=x.dtype)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib().mf_merge_heads(_ptr_array([x]), None, packed.data_ptr(), 1, B, N, H, D,
                                                 _CODE[x.dtype], _stream(x.device)))  # fmt: skip
        ctx.meta = (B, H, N, D)
        return packed

    @staticmethod
    def backward(ctx, g):
        B, H, N, D = ctx.meta
        g = g.contiguous()
        out = torch.empty((B, H, N, D), device=g.device, dtype=g.dtype)
        with torch.cuda.device(g.device):
            _lib.check(_lib.lib().mf_split_heads(g.data_ptr(), _ptr_array([out]), None, 1, B, N, H, D, _CODE[g.dtype],
                                                 _stream(g.device)))  # fmt: skip
        return out


def split_heads(packed: torch.Tensor, groups: int, heads: int, scales=None):
    """(B, N, groups*heads*D) -> ``groups`` contiguous tensors (B, heads, N, D); group g multiplied by ``scales[g]``."""
    return _SplitHeads.apply(packed, groups, heads, tuple(scales) if scales is not None else None)


def merge_heads(x: torch.Tensor) -> torch.Tensor:
    """(B, H, N, D) -> (B, N, H*D)."""
    return _MergeHeads.apply(x)


PAIR_HIDDEN, PAIR_RBF = 128, 16


def pair_head_applies(a: torch.Tensor, w_rbf: torch.Tensor) -> bool:
    """The coordinate-head kernel is built for a 128-wide pair MLP with 16 radial basis functions on CUDA fp32 / bf16."""
    return (a.is_cuda and a.dtype in _CODE and a.ndim == 3 and a.shape[-1] == PAIR_HIDDEN
            and tuple(w_rbf.shape) == (PAIR_HIDDEN, PAIR_RBF))  # fmt: skip


class _PairHead(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, coords, valid, w_rbf, w_out, b_out, centers, gamma):
        ctx.param_dtypes = (w_rbf.dtype, w_out.dtype, b_out.dtype)
        ctx.w_out_shape, ctx.b_out_shape = tuple(w_out.shape), tuple(b_out.shape)
        a = a.contiguous()
        b = b.to(a.dtype).contiguous()
        coords = coords.detach().float().contiguous()
        valid = valid.to(torch.uint8).contiguous()
        w_rbf, w_out = w_rbf.detach().float().contiguous(), w_out.detach().float().reshape(-1).contiguous()
        b_out, centers = b_out.detach().float().reshape(-1).contiguous(), centers.detach().float().contiguous()
        B, N, _ = a.shape
        out = torch.empty((B, N, 3), device=a.device, dtype=torch.float32)
        args = _lib.MfPairHeadArgs(batch=B, tokens=N, hidden=PAIR_HIDDEN, n_rbf=PAIR_RBF, dtype=_CODE[a.dtype],
                                   gamma=float(gamma), a=a.data_ptr(), b=b.data_ptr(), coords=coords.data_ptr(),
                                   valid=valid.data_ptr(), w_rbf=w_rbf.data_ptr(), w_out=w_out.data_ptr(),
                                   b_out=b_out.data_ptr(), centers=centers.data_ptr(), out=out.data_ptr())  # fmt: skip
        with torch.cuda.device(a.device):
            _lib.check(_lib.lib().mf_pair_head_fwd(ctypes.byref(args), _stream(a.device)))
        ctx.save_for_backward(a, b, coords, valid, w_rbf, w_out, b_out, centers)
        ctx.gamma = float(gamma)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        a, b, coords, valid, w_rbf, w_out, b_out, centers = ctx.saved_tensors
        B, N, _ = a.shape
        grad_out = grad_out.float().contiguous()
        da, db = torch.empty_like(a), torch.empty_like(b)
        dparams = torch.empty(PAIR_HIDDEN * PAIR_RBF + PAIR_HIDDEN + 4, device=a.device, dtype=torch.float32)
        d_w_rbf = dparams[: PAIR_HIDDEN * PAIR_RBF].view(PAIR_HIDDEN, PAIR_RBF)
        d_w_out = dparams[PAIR_HIDDEN * PAIR_RBF : PAIR_HIDDEN * PAIR_RBF + PAIR_HIDDEN]
        d_b_out = dparams[PAIR_HIDDEN * PAIR_RBF + PAIR_HIDDEN : PAIR_HIDDEN * PAIR_RBF + PAIR_HIDDEN + 1]
        args = _lib.MfPairHeadArgs(batch=B, tokens=N, hidden=PAIR_HIDDEN, n_rbf=PAIR_RBF, dtype=_CODE[a.dtype],
                                   gamma=ctx.gamma, a=a.data_ptr(), b=b.data_ptr(), coords=coords.data_ptr(),
                                   valid=valid.data_ptr(), w_rbf=w_rbf.data_ptr(), w_out=w_out.data_ptr(),
                                   b_out=b_out.data_ptr(), centers=centers.data_ptr(), grad_out=grad_out.data_ptr(),
                                   grad_a=da.data_ptr(), grad_b=db.data_ptr(), grad_w_rbf=d_w_rbf.data_ptr(),
                                   grad_w_out=d_w_out.data_ptr(), grad_b_out=d_b_out.data_ptr())  # fmt: skip
        with torch.cuda.device(a.device):
            need = int(_lib.lib().mf_pair_head_bwd_workspace_bytes(ctypes.byref(args)))
            ws = torch.empty(max(need, 16), device=a.device, dtype=torch.uint8)
            args.workspace, args.workspace_bytes = ws.data_ptr(), need
            _lib.check(_lib.lib().mf_pair_head_bwd(ctypes.byref(args), _stream(a.device)))
        dt = ctx.param_dtypes
        return (da, db, None, None, d_w_rbf.to(dt[0]), d_w_out.reshape(ctx.w_out_shape).to(dt[1]),
                d_b_out.reshape(ctx.b_out_shape).to(dt[2]), None, None)  # fmt: skip


def equivariant_pair_head(a: torch.Tensor, b: torch.Tensor, coords: torch.Tensor, valid: torch.Tensor,
                          w_rbf: torch.Tensor, w_out: torch.Tensor, b_out: torch.Tensor, centers: torch.Tensor,
                          gamma: float) -> torch.Tensor:  # fmt: skip
    """Coordinate update of ``QM9EDMModel._equivariant_coord_delta`` (src/matterformer/models/qm9.py:478-501).

    ``a`` / ``b`` (B, N, 128): the pair MLP's first Linear applied to the trunk output, split into its ``h_i`` and
    ``h_j`` column blocks (the bias goes with ``b``); ``w_rbf`` (128, 16) its radial-basis columns; ``w_out`` / ``b_out``
    the second Linear; ``coords`` (B, N, 3), ``valid`` (B, N) bool.  Returns (B, N, 3) fp32: per atom the weighted sum
    of displacements to the molecule's other real atoms, divided by their number, minus its mean over the molecule.
    Gradients flow to ``a``, ``b``, ``w_rbf``, ``w_out`` and ``b_out``; the coordinates are treated as data.
    """
    return _PairHead.apply(a, b, coords, valid, w_rbf, w_out, b_out, centers, gamma)
