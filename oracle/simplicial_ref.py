"""CPU restatement of Matterformer's dense 2-simplicial attention (TEST INFRASTRUCTURE).

This module is the parity oracle for the CUDA kernels.  It is imported only by
``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline / reference
legs of ``bench.py``; the product package never imports it.

It restates, in plain torch on the CPU, the algorithm of the reference's
``simplicial_attention_torch_from_projected``
(src/matterformer/models/simplicial_attention.py:206-344):

* logits[b,h,i,j,k] = sum_d k1[b,h,j,d] * (q[b,h,i,d] * k2[b,h,k,d])
  (``_materialize_chunk_logits``, simplicial_attention.py:161-180), cast to fp32;
* + gate_i * (u_ij + v_ik + w_jk)           (``SimplicialFactorizedBias.chunk``, :41-47)
* + gate_i * R^-1/2 * sum_r L_ijr * R_ikr    (``SimplicialLowRankAngleResidual.chunk``, :76-81)
* pair (j,k) is visible iff key_valid[j] & key_valid[k] & pair_valid[j,k]
  (``SimplicialAttentionMask.pair_mask``, :141-145); masked logits are filled
  with finfo.min, softmax runs over the flattened (j,k) axis and masked
  probabilities are then forced to zero (:317-319), so a query with no visible
  pair returns zero;
* out[b,h,i,d] = sum_jk attn[i,j,k] * v1[j,d] * v2[k,d]  (:326-329)
* + R^-1/2 * sum_jk attn * L_ijr * R_ikr  contracted with message_basis[h,r,d] (:330-337)
* rows of invalid queries are zeroed (:338-339).

Parity of this restatement is pinned by the golden vectors under
``tests/golden/`` which were produced by the reference implementation itself
(see ``tests/golden/make_golden.py``) and by the reference's known-answer test
(tests/test_simplicial_attention.py:448-463) restated in ``tests/test_oracle.py``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class SimplicialInputs:
    """Everything the reference's autograd boundary receives (simplicial_attention.py:349-372)."""

    q: torch.Tensor
    k1: torch.Tensor
    v1: torch.Tensor
    k2: torch.Tensor
    v2: torch.Tensor
    query_valid: torch.Tensor  # (B, N) bool
    pair_key_valid: torch.Tensor  # (B, N) bool
    pair_valid: Optional[torch.Tensor] = None  # (B, N, N) bool
    u: Optional[torch.Tensor] = None  # (B, H, N, N)
    v_bias: Optional[torch.Tensor] = None
    w: Optional[torch.Tensor] = None
    gate: Optional[torch.Tensor] = None  # (B, H, N)
    angle_left: Optional[torch.Tensor] = None  # (B, H, N, N, R)
    angle_right: Optional[torch.Tensor] = None
    angle_gate: Optional[torch.Tensor] = None  # (B, H, N)
    message_left: Optional[torch.Tensor] = None  # (B, H, N, N, R)
    message_right: Optional[torch.Tensor] = None
    message_basis: Optional[torch.Tensor] = None  # (H, R, D)


def pair_mask(inp: SimplicialInputs) -> torch.Tensor:
    """(B, N, N) visibility of the key pair (j, k); simplicial_attention.py:141-145."""
    kv = inp.pair_key_valid.bool()
    m = kv[:, :, None] & kv[:, None, :]
    if inp.pair_valid is not None:
        m = m & inp.pair_valid.bool()
    return m


def simplicial_forward(inp: SimplicialInputs, *, fp32_core: bool = True, return_lse: bool = False):
    """Forward pass for one batch, looping over batch elements to bound memory.

    ``fp32_core=True`` upcasts every operand to fp32 first (simplicial_attention.py:251-297);
    ``False`` keeps matmuls in the input dtype like the reference's default path, which for
    bf16 inputs rounds the logits to bf16 before the fp32 softmax (:173).
    Returns ``out`` in fp32 (fp32_core) or the dtype of ``v1``; with ``return_lse`` also the
    log-sum-exp over visible pairs (0 where the query is invalid or sees no pair), which is what
    the reference's kernel interface saves for backward (triton_simplicial_attention.py:316-329).
    """
    q, k1, v1, k2, v2 = inp.q, inp.k1, inp.v1, inp.k2, inp.v2
    if fp32_core:
        q, k1, v1, k2, v2 = (t.float() for t in (q, k1, v1, k2, v2))
    B, H, N, D = q.shape
    mask = pair_mask(inp)
    outs = []
    lses = []
    for b in range(B):
        qk2 = q[b, :, :, None, :] * k2[b, :, None, :, :]  # (H, i, k, D)
        logits = torch.einsum("hjd,hikd->hijk", k1[b], qk2).float()
        if inp.u is not None:
            g = inp.gate[b].float()[:, :, None, None]
            bias = (
                inp.u[b].float()[:, :, :, None]
                + inp.v_bias[b].float()[:, :, None, :]
                + inp.w[b].float()[:, None, :, :]
            )
            logits = logits + g * bias
        if inp.angle_left is not None:
            rank = inp.angle_left.shape[-1]
            res = torch.einsum("hijr,hikr->hijk", inp.angle_left[b].float(), inp.angle_right[b].float()) * rank**-0.5
            logits = logits + inp.angle_gate[b].float()[:, :, None, None] * res
        m = mask[b][None, None, :, :].expand(H, N, N, N)
        flat = logits.masked_fill(~m, torch.finfo(torch.float32).min).flatten(-2)
        attn = torch.softmax(flat, dim=-1)
        attn = torch.where(m.flatten(-2), attn, torch.zeros_like(attn)).view(H, N, N, N)
        a = attn.to(v1.dtype)
        tmp = torch.einsum("hijk,hjd->hikd", a, v1[b])
        out = (tmp * v2[b][:, None, :, :]).sum(dim=-2)
        if inp.message_left is not None:
            rank = inp.message_left.shape[-1]
            coeff = torch.einsum(
                "hijk,hijr,hikr->hir", attn.float(), inp.message_left[b].float(), inp.message_right[b].float()
            ) * rank**-0.5
            out = out + torch.einsum("hir,hrd->hid", coeff, inp.message_basis.float()).to(out.dtype)
        qv = inp.query_valid[b].to(out.dtype)
        out = out * qv[None, :, None]
        outs.append(out)
        if return_lse:
            neg_inf = torch.full_like(logits, float("-inf"))
            lse = torch.logsumexp(torch.where(m, logits, neg_inf).flatten(-2), dim=-1)
            any_pair = m.flatten(-2).any(dim=-1)
            lse = torch.where(any_pair & inp.query_valid[b][None, :], lse, torch.zeros_like(lse))
            lses.append(lse)
    out = torch.stack(outs, 0)
    if return_lse:
        return out, torch.stack(lses, 0)
    return out


_GRAD_FIELDS = (
    "q",
    "k1",
    "v1",
    "k2",
    "v2",
    "u",
    "v_bias",
    "w",
    "gate",
    "angle_left",
    "angle_right",
    "angle_gate",
    "message_left",
    "message_right",
    "message_basis",
)


def simplicial_forward_backward(inp: SimplicialInputs, grad_out: torch.Tensor, *, fp32_core: bool = True):
    """Returns (out, {name: grad}) by autograd through :func:`simplicial_forward`.

    Mirrors how the reference derives its own check gradients
    (simplicial_attention.py:454-552: autograd through the torch path with fp32_core=True).
    """
    fields = {}
    leaves = []
    names = []
    for name in _GRAD_FIELDS:
        t = getattr(inp, name)
        if t is None:
            continue
        t = t.detach().clone().requires_grad_(True)
        fields[name] = t
        leaves.append(t)
        names.append(name)
    work = SimplicialInputs(
        **fields,
        query_valid=inp.query_valid,
        pair_key_valid=inp.pair_key_valid,
        pair_valid=inp.pair_valid,
    )
    out = simplicial_forward(work, fp32_core=fp32_core)
    grads = torch.autograd.grad(out, leaves, grad_out.to(out.dtype), allow_unused=True)
    return out.detach(), {n: (g if g is not None else torch.zeros_like(fields[n])) for n, g in zip(names, grads)}
