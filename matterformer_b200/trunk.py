"""Dense-token trunk and EDM denoising step around the attention kernels.

A lean, self-contained mirror of the reference modules that call the attention hot path, so that
the trunk workload (12 layers alternating MHA and 2-simplicial attention, d_model 512, 8 heads) can
run where the reference package is not installed.  Module and parameter names follow the reference,
so a reference ``state_dict`` of the same configuration loads with ``strict=True``:

* :class:`SimplicialAttention`  <- src/matterformer/models/simplicial_attention.py:640-987
  (5-way ``in_proj`` in the order q,k1,v1,k2,v2, ``q *= head_dim**-0.5``, ``out_proj``)
* :class:`RegularAttention`     <- src/matterformer/models/regular_attention.py:275-338 (``nn.MultiheadAttention``)
* :class:`AdaLNBlock`, :class:`Mlp`, :class:`TransformerTrunk` <- src/matterformer/models/transformer.py:129-316, 1062-1317
* :class:`TimeEmbedder`         <- src/matterformer/models/embeddings.py:9-44
* :class:`EDMModel`             <- ``QM9EDMModel`` with geometry bias off, src/matterformer/models/qm9.py:249-565
* :class:`EDMPreconditioner`, :class:`EDMLoss` <- src/matterformer/tasks/edm.py:34-150

Only what that configuration touches is mirrored: no geometry-bias builders, no RoPE, no coordinate
embedding.  ``impl="cuda"`` (and ``"auto"`` on CUDA tensors) runs the sm_100a kernels through the C ABI;
``impl="torch"`` is the dense formulation in plain torch ops, as in the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch
import torch.nn.functional as F
from torch import nn

from . import fused
from .fused import (fused_applies, gated_residual, heads_layout_applies, ln_modulate, merge_heads, split_heads,
                    split_modulation)
from .linear import linear_bf16, linear_gelu_bf16, refresh_bf16_copies
from .simplicial import (normalize_simplicial_precision, packed_projection_applies, simplicial_attention_cuda,
                         simplicial_attention_packed)  # fmt: skip


@dataclass(frozen=True)
class SimplicialAttentionMask:
    """ref: SimplicialAttentionMask, simplicial_attention.py:107-145."""

    query_valid: torch.Tensor
    pair_key_valid: torch.Tensor
    pair_valid: Optional[torch.Tensor] = None

    @classmethod
    def from_key_padding_mask(cls, key_padding_mask, *, batch_size: int, num_tokens: int, device):
        if key_padding_mask is None:
            valid = torch.ones(batch_size, num_tokens, device=device, dtype=torch.bool)
        else:
            if key_padding_mask.shape != (batch_size, num_tokens):
                raise ValueError(
                    f"key_padding_mask must have shape {(batch_size, num_tokens)}, got {tuple(key_padding_mask.shape)}"
                )
            valid = ~key_padding_mask.bool().to(device=device)
        return cls(query_valid=valid, pair_key_valid=valid)

    def pair_mask(self) -> torch.Tensor:
        m = self.pair_key_valid[:, :, None] & self.pair_key_valid[:, None, :]
        if self.pair_valid is not None:
            m = m & self.pair_valid.bool()
        return m


def simplicial_attention_dense_torch(q, k1, v1, k2, v2, mask: SimplicialAttentionMask) -> torch.Tensor:
    """The dense torch formulation (logits over all (j,k), fp32 softmax); used by ``impl="torch"``."""
    pair = mask.pair_mask()[:, None, None, :, :]
    logits = torch.einsum("bhjd,bhikd->bhijk", k1, q[:, :, :, None, :] * k2[:, :, None, :, :]).float()
    flat = logits.flatten(-2).masked_fill(~pair.flatten(-2), torch.finfo(torch.float32).min)
    attn = torch.softmax(flat, dim=-1)
    attn = torch.where(pair.flatten(-2), attn, torch.zeros_like(attn)).view_as(logits).to(v1.dtype)
    out = (torch.einsum("bhijk,bhjd->bhikd", attn, v1) * v2[:, :, None, :, :]).sum(dim=-2)
    return out * mask.query_valid[:, None, :, None].to(out.dtype)


class SimplicialAttention(nn.Module):
    """Dense non-causal 2-simplicial attention layer (projections + kernel + output projection)."""

    def __init__(self, dim: int, num_heads: int, *, head_dim: Optional[int] = None, bias: bool = True,
                 impl: str = "auto", precision: str = "bf16_tc") -> None:  # fmt: skip
        super().__init__()
        if head_dim is None:
            if dim % num_heads != 0:
                raise ValueError(f"dim ({dim}) must be divisible by num_heads ({num_heads}) when head_dim is None.")
            head_dim = dim // num_heads
        impl = impl.lower()
        if impl == "triton":  # the reference's name for "the kernel backend"
            impl = "cuda"
        if impl not in {"auto", "torch", "cuda"}:
            raise ValueError(f"Unsupported simplicial_impl: {impl}")
        self.dim, self.num_heads, self.head_dim = int(dim), int(num_heads), int(head_dim)
        self.inner_dim = self.num_heads * self.head_dim
        self.impl = impl
        self.precision = normalize_simplicial_precision(precision)
        self.scale = self.head_dim**-0.5
        self._last_impl_used = "torch"
        self.in_proj = nn.Linear(self.dim, 5 * self.inner_dim, bias=bias)
        self.out_proj = nn.Linear(self.inner_dim, self.dim, bias=bias)

    def _split(self, t: torch.Tensor) -> torch.Tensor:
        b, n, _ = t.shape
        return t.view(b, n, self.num_heads, self.head_dim).transpose(1, 2)

    def _project_out(self, out: torch.Tensor) -> torch.Tensor:
        if not torch.is_autocast_enabled() and out.dtype != torch.bfloat16:
            out = out.to(self.out_proj.weight.dtype)
        return linear_bf16(out, self.out_proj.weight, self.out_proj.bias)

    def forward(self, x: torch.Tensor, *, key_padding_mask: Optional[torch.Tensor] = None,
                attention_mask: Optional[SimplicialAttentionMask] = None) -> torch.Tensor:  # fmt: skip
        if x.ndim != 3:
            raise ValueError(f"x must have shape (B, T, C), got {tuple(x.shape)}")
        b, n, _ = x.shape
        if attention_mask is None:
            attention_mask = SimplicialAttentionMask.from_key_padding_mask(
                key_padding_mask, batch_size=b, num_tokens=n, device=x.device
            )
        on_gpu = x.device.type == "cuda"
        if self.impl == "cuda" and not on_gpu:
            raise RuntimeError("CUDA simplicial attention is unavailable: the CUDA backend requires CUDA tensors")
        use_cuda = self.impl == "cuda" or (self.impl == "auto" and on_gpu)
        self._last_impl_used = "cuda" if use_cuda else "torch"
        proj = linear_bf16(x, self.in_proj.weight, self.in_proj.bias)
        dtype = torch.bfloat16 if self.precision == "bf16_tc" else torch.float32
        if use_cuda and self.precision == "bf16_tc" and packed_projection_applies(proj, self.num_heads, self.head_dim):
            # small molecules: the kernels read q, k1, v1, k2, v2 where the GEMM left them and write what out_proj reads
            out = simplicial_attention_packed(proj, heads=self.num_heads, query_valid=attention_mask.query_valid,
                                              pair_key_valid=attention_mask.pair_key_valid,
                                              pair_valid=attention_mask.pair_valid, q_scale=self.scale)  # fmt: skip
            return self._project_out(out)
        if use_cuda and heads_layout_applies(proj, self.num_heads, 5):
            # one pass from the projection's (B, N, 5, H, D) to the five head-major tensors, queries scaled on the way
            q, k1, v1, k2, v2 = split_heads(proj.to(dtype), 5, self.num_heads, (self.scale, 1.0, 1.0, 1.0, 1.0))
            out = simplicial_attention_cuda(
                q, k1, v1, k2, v2, query_valid=attention_mask.query_valid,
                pair_key_valid=attention_mask.pair_key_valid, pair_valid=attention_mask.pair_valid,
                precision=self.precision,
            )  # fmt: skip
            out = merge_heads(out)
            return self._project_out(out)
        q, k1, v1, k2, v2 = (self._split(t) for t in proj.chunk(5, dim=-1))
        q = q * self.scale
        if use_cuda:
            out = simplicial_attention_cuda(
                q.to(dtype), k1.to(dtype), v1.to(dtype), k2.to(dtype), v2.to(dtype),
                query_valid=attention_mask.query_valid, pair_key_valid=attention_mask.pair_key_valid,
                pair_valid=attention_mask.pair_valid, precision=self.precision,
            )  # fmt: skip
        else:
            out = simplicial_attention_dense_torch(q, k1, v1, k2, v2, attention_mask)
        out = out.transpose(1, 2).reshape(b, n, self.inner_dim)
        return self._project_out(out)


@dataclass
class SparseAttentionPlan:
    """What the MHA layers of a periodic trunk attend over.  Built once per step from the structure (positions and
    lattice do not change between layers) and handed to every MHA layer, the way the reference hands one additive
    ``(B, H, T, T)`` mask to every block (AdaLNBlock.forward, src/matterformer/models/transformer.py:254-268).

    ``kind="radius"``: pairs within ``blocks.cutoff`` under the minimum-image convention (self included), through
    :func:`radius_block_sparse_attention`.  ``kind="local"``: a band of ``window`` tokens in the cell-sorted order of
    ``blocks.perm`` (atoms of one grid cell are neighbours in that order), through :func:`local_window_attention`.
    """

    kind: str
    blocks: "RadiusBlocks"
    num_atoms: torch.Tensor
    window: int = 64


def plan_sparse_attention(frac: torch.Tensor, lattice: torch.Tensor, pad_mask: Optional[torch.Tensor], cutoff: float,
                          kind: str = "radius", window: int = 64) -> SparseAttentionPlan:  # fmt: skip
    """Cell-sorts the atoms and lists the active tiles (one pass over the structure; no gradient flows through it).

    ``frac`` (B, N, 3) fractional coordinates, ``lattice`` (B, 6) latent or (B, 3, 3) cell, ``pad_mask`` (B, N) with
    True on padded tokens, which must form a suffix of every row.
    """
    from .sparse import build_radius_blocks

    if kind not in {"radius", "local"}:
        raise ValueError(f"Unsupported sparse attention kind: {kind}")
    b, n, _ = frac.shape
    if pad_mask is None:
        num_atoms = torch.full((b,), n, dtype=torch.int32, device=frac.device)
    else:
        num_atoms = (~pad_mask.bool()).sum(dim=1).to(torch.int32)
    blocks = build_radius_blocks(frac.detach(), lattice.detach(), num_atoms, float(cutoff))
    return SparseAttentionPlan(kind=kind, blocks=blocks, num_atoms=num_atoms, window=int(window))


class RegularAttention(nn.Module):
    """Standard multi-head self-attention (``position_mode="none"`` of the reference wrapper,
    regular_attention.py:275-338); parameters are those of ``nn.MultiheadAttention``.

    ``impl="auto"`` runs the attention core on this library's local-window kernel when that is the
    same computation: CUDA, bf16 (autocast or bf16 input), at most 32 tokens (a window of 64 then
    covers every pair), head size 32/64/128, no active dropout, and a key-padding mask that marks a
    suffix of every row (how the reference's collate functions pad, data/qm9.py:119-166).  The suffix
    property is verified on the device once per mask tensor (one read-back, remembered for the other
    layers of the step; a mask first seen while a CUDA graph is being captured cannot be read back
    and is taken to be the one checked during the eager warm-up steps).  A mask with holes goes to
    ``nn.MultiheadAttention`` like everything else this kernel does not cover.  Rows of padded tokens
    return zeros on the kernel path instead of the reference's average over the real keys; the trunk
    discards those rows.  ``impl="torch"`` always uses ``nn.MultiheadAttention``.
    """

    def __init__(self, embed_dim: int, num_heads: int, *, dropout: float = 0.0, impl: str = "auto") -> None:
        super().__init__()
        if impl not in {"auto", "torch"}:
            raise ValueError(f"Unsupported attention impl: {impl}")
        self.attn = nn.MultiheadAttention(embed_dim, num_heads, dropout=dropout, batch_first=True)
        self.impl = impl
        self._last_core_used: Optional[str] = None

    _suffix_cache: tuple = (None, True)  # (identity of the last mask checked, result); shared by all layers

    @classmethod
    def _padding_is_a_suffix(cls, mask: torch.Tensor) -> bool:
        key = (mask.data_ptr(), mask._version, tuple(mask.shape))
        if cls._suffix_cache[0] == key:
            return cls._suffix_cache[1]
        if torch.cuda.is_current_stream_capturing():
            return True
        ok = bool((mask[:, 1:] | ~mask[:, :-1]).all().item()) if mask.shape[1] > 1 else True
        cls._suffix_cache = (key, ok)
        return ok

    def _cuda_core_applies(self, x: torch.Tensor, key_padding_mask: Optional[torch.Tensor]) -> bool:
        if self.impl == "torch" or not x.is_cuda or key_padding_mask is None or x.shape[1] > 32:
            return False
        if self.training and self.attn.dropout > 0.0:
            return False
        bf16 = x.dtype == torch.bfloat16 or (
            torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16
        )
        if not (bf16 and (self.attn.embed_dim // self.attn.num_heads) in (32, 64, 128)):
            return False
        return self._padding_is_a_suffix(key_padding_mask)

    def _sparse_forward(self, x: torch.Tensor, plan: SparseAttentionPlan) -> torch.Tensor:
        """The layer with its core on the radius block-sparse or the local-window kernel.  Same parameters and
        projections as the dense layer; only the set of visible keys differs."""
        from .sparse import local_window_attention, radius_block_sparse_attention

        H = self.attn.num_heads
        low = x.dtype == torch.bfloat16 or (torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16)
        qkv = F.linear(x, self.attn.in_proj_weight, self.attn.in_proj_bias)
        qkv = qkv.to(torch.bfloat16) if low else qkv.float()
        q, k, v = split_heads(qkv, 3, H)  # each (B, H, N, D), one pass
        if plan.kind == "radius":
            core = radius_block_sparse_attention(q, k, v, plan.blocks, sorted_inputs=False)
        else:  # band over the cell-sorted order: gather, attend, scatter back
            idx = plan.blocks.perm.long()[:, None, :, None].expand_as(q)
            qs, ks, vs = (torch.gather(t, 2, idx) for t in (q, k, v))
            core = torch.zeros_like(q).scatter(2, idx, local_window_attention(qs, ks, vs, plan.num_atoms, window=plan.window))
        self._last_core_used = plan.kind
        return self.attn.out_proj(merge_heads(core))

    def forward(self, x: torch.Tensor, *, key_padding_mask: Optional[torch.Tensor] = None,
                sparse_plan: Optional[SparseAttentionPlan] = None) -> torch.Tensor:  # fmt: skip
        if sparse_plan is not None:
            if not x.is_cuda:
                raise RuntimeError("sparse attention plans need CUDA tensors (there is no CPU fallback)")
            return self._sparse_forward(x, sparse_plan)
        if not self._cuda_core_applies(x, key_padding_mask):
            self._last_core_used = "torch"
            out, _ = self.attn(x, x, x, key_padding_mask=key_padding_mask, need_weights=False)
            return out
        from .sparse import local_window_attention_packed

        self._last_core_used = "cuda"
        B, N, C = x.shape
        H = self.attn.num_heads
        qkv = linear_bf16(x, self.attn.in_proj_weight, self.attn.in_proj_bias).to(torch.bfloat16)
        num_atoms = (~key_padding_mask).sum(dim=1).to(torch.int32)
        # with at most 32 tokens the window-64 band covers every real token: dense attention, straight on the projection
        core = local_window_attention_packed(qkv, H, num_atoms, window=64)
        return linear_bf16(core, self.attn.out_proj.weight, self.attn.out_proj.bias)


class Mlp(nn.Module):
    def __init__(self, d_model: int, mlp_ratio: float = 4.0) -> None:
        super().__init__()
        hidden = int(d_model * mlp_ratio)
        self.fc1 = nn.Linear(d_model, hidden)
        self.act = nn.GELU(approximate="tanh")
        self.fc2 = nn.Linear(hidden, d_model)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear_bf16(linear_gelu_bf16(x, self.fc1.weight, self.fc1.bias), self.fc2.weight, self.fc2.bias)


def layer_norm(x: torch.Tensor, norm: nn.LayerNorm) -> torch.Tensor:
    """``norm(x)`` for a (B, N, C) CUDA tensor through the fused LayerNorm-modulate kernels (ATen's backward for an
    affine LayerNorm of this width is ten times slower than its forward): the affine weight and bias become the
    modulation ``scale = weight - 1``, ``shift = bias`` of every molecule, and their gradients come back through the
    broadcast.  Other tensors take ``norm`` itself."""
    if not (fused_applies(x) and x.dtype == torch.float32 and norm.normalized_shape == (x.shape[-1],)):
        return norm(x)
    B, C = x.shape[0], x.shape[-1]
    if norm.elementwise_affine:
        scale = (norm.weight.float() - 1.0).expand(B, C)
        shift = (norm.bias.float() if norm.bias is not None else torch.zeros_like(norm.weight, dtype=torch.float32)).expand(B, C)
    else:
        scale = shift = torch.zeros((B, C), device=x.device, dtype=torch.float32)
    return ln_modulate(x, shift, scale, eps=norm.eps, out_dtype=torch.float32)


def _modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return x * (1.0 + scale[:, None, :]) + shift[:, None, :]


class AdaLNBlock(nn.Module):
    """Pre-norm block with adaptive LayerNorm conditioning and gated residuals (transformer.py:154-316)."""

    def __init__(self, d_model: int, n_heads: int, *, mlp_ratio: float = 4.0, eps: float = 1e-6,
                 attn_type: str = "mha", simplicial_impl: str = "auto", simplicial_precision: str = "bf16_tc") -> None:  # fmt: skip
        super().__init__()
        attn_type = attn_type.lower()
        if attn_type not in {"mha", "simplicial"}:
            raise ValueError(f"Unsupported attn_type: {attn_type}")
        self.attn_type = attn_type
        self.norm1 = nn.LayerNorm(d_model, eps=eps, elementwise_affine=False)
        self.norm2 = nn.LayerNorm(d_model, eps=eps, elementwise_affine=False)
        self.ada_ln = nn.Sequential(nn.SiLU(), nn.Linear(d_model, 6 * d_model, bias=True))
        nn.init.zeros_(self.ada_ln[-1].weight)
        nn.init.zeros_(self.ada_ln[-1].bias)
        if attn_type == "mha":
            self.attn = RegularAttention(d_model, n_heads)
        else:
            self.attn = SimplicialAttention(d_model, n_heads, impl=simplicial_impl, precision=simplicial_precision)
        self.mlp = Mlp(d_model, mlp_ratio)
        self.fused_elementwise = True  # CUDA fp32 residual stream: fused norm+modulate and gated-residual kernels

    def forward(self, x, cond_emb, *, pad_mask=None, simplicial_attention_mask=None, sparse_plan=None,
                zero_padding: bool = False, cond_act=None):
        """``zero_padding``: return the block's output with its padded rows cleared (the ``masked_fill`` the trunk
        applies before the next block), folded into the last fused pass when the fused kernels run.  ``cond_act``:
        ``SiLU(cond_emb)`` when the caller has already formed it (it is the same for every block of a trunk)."""
        mod = linear_bf16(cond_act if cond_act is not None else self.ada_ln[0](cond_emb), self.ada_ln[-1].weight,
                          self.ada_ln[-1].bias)  # fmt: skip
        fused = self.fused_elementwise and fused_applies(x)
        shift_a, scale_a, gate_a, shift_m, scale_m, gate_m = split_modulation(mod) if fused else mod.chunk(6, dim=-1)
        if fused:
            # one pass each for norm + modulate and for the gated residual; under bf16 autocast the modulated
            # activations are written in bf16, which is what the Linear layers that consume them cast to anyway
            low = torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16
            h_dtype = torch.bfloat16 if (low or x.dtype == torch.bfloat16) else torch.float32
            h = ln_modulate(x, shift_a, scale_a, eps=self.norm1.eps, out_dtype=h_dtype)
        else:
            h = _modulate(self.norm1(x), shift_a, scale_a)
        if self.attn_type == "mha":
            attn_out = self.attn(h, key_padding_mask=pad_mask, sparse_plan=sparse_plan)
        else:
            attn_out = self.attn(h, key_padding_mask=pad_mask, attention_mask=simplicial_attention_mask)
        if fused:
            x = gated_residual(x, gate_a, attn_out)
            h = ln_modulate(x, shift_m, scale_m, eps=self.norm2.eps, out_dtype=h_dtype)
            return gated_residual(x, gate_m, self.mlp(h), pad_mask if zero_padding else None)
        x = x + gate_a[:, None, :] * attn_out
        h = _modulate(self.norm2(x), shift_m, scale_m)
        x = x + gate_m[:, None, :] * self.mlp(h)
        return x.masked_fill(pad_mask[..., None], 0.0) if (zero_padding and pad_mask is not None) else x


class TransformerTrunk(nn.Module):
    """Stack of :class:`AdaLNBlock`; ``attn_types`` names the attention of every layer, e.g. alternating."""

    def __init__(self, d_model: int, n_heads: int, attn_types: Sequence[str], *, mlp_ratio: float = 4.0,
                 eps: float = 1e-6, simplicial_impl: str = "auto", simplicial_precision: str = "bf16_tc",
                 emit_pair_valid: bool = True) -> None:  # fmt: skip
        super().__init__()
        self.blocks = nn.ModuleList(
            AdaLNBlock(d_model, n_heads, mlp_ratio=mlp_ratio, eps=eps, attn_type=t, simplicial_impl=simplicial_impl,
                       simplicial_precision=simplicial_precision)  # fmt: skip
            for t in attn_types
        )
        self.norm_out = nn.LayerNorm(d_model, eps=eps, elementwise_affine=False)
        # The reference hands the kernel a dense (B,T,T) pair mask whenever a geometry adapter exists
        # (transformer.py:36-73), even though it only repeats the padding; keep that behaviour by default.
        self.emit_pair_valid = bool(emit_pair_valid)

    def _linear_parameters(self):
        """Weights and biases of the blocks' Linear layers (the ones :func:`linear_bf16` serves)."""
        out = []
        for block in self.blocks:
            attn = block.attn.attn if isinstance(block.attn, RegularAttention) else block.attn
            layers = [block.ada_ln[-1], block.mlp.fc1, block.mlp.fc2, attn.out_proj]
            out += [p for layer in layers for p in (layer.weight, layer.bias)]
            out += [attn.in_proj_weight, attn.in_proj_bias] if isinstance(block.attn, RegularAttention) else \
                   [attn.in_proj.weight, attn.in_proj.bias]  # fmt: skip
        return out

    def forward(self, x: torch.Tensor, cond_emb: torch.Tensor, *, pad_mask: Optional[torch.Tensor] = None,
                sparse_plan: Optional[SparseAttentionPlan] = None) -> torch.Tensor:  # fmt: skip
        """``sparse_plan`` (see :func:`plan_sparse_attention`) makes every MHA layer attend over the plan's
        neighbourhoods instead of all tokens: the periodic-crystal mode of the trunk."""
        b, n, _ = x.shape
        if pad_mask is not None:
            pad_mask = pad_mask.bool()
        if x.is_cuda and torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16:
            # the bf16 copies the blocks' Linear layers compute with: all of them in one multi-tensor copy; a step that is
            # being captured into a CUDA graph always contains the copy (its replays change the parameters)
            refresh_bf16_copies(self._linear_parameters(), force=torch.cuda.is_current_stream_capturing())
        sim_mask = SimplicialAttentionMask.from_key_padding_mask(pad_mask, batch_size=b, num_tokens=n, device=x.device)
        if self.emit_pair_valid:
            v = sim_mask.pair_key_valid
            sim_mask = SimplicialAttentionMask(sim_mask.query_valid, v, v[:, :, None] & v[:, None, :])
        # the reference clears the padded rows before every block (transformer.py, the loop of TransformerTrunk.forward);
        # here every block hands its output over already cleared (one pass with its last gated residual), which is
        # the same for every block but the last, whose padded rows are cleared once more after the output norm anyway
        if pad_mask is not None:
            x = x.masked_fill(pad_mask[..., None], 0.0)
        # every block starts its modulation with the same SiLU(cond_emb): formed (and cast for the bf16 Linear) once
        cond_act = F.silu(cond_emb)
        if x.is_cuda and torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16:
            cond_act = cond_act.to(torch.bfloat16)
        for block in self.blocks:
            x = block(x, cond_emb, pad_mask=pad_mask, simplicial_attention_mask=sim_mask, sparse_plan=sparse_plan,
                      zero_padding=pad_mask is not None, cond_act=cond_act)
        x = layer_norm(x, self.norm_out)
        if pad_mask is not None:
            x = x.masked_fill(pad_mask[..., None], 0.0)
        return x


class TimeEmbedder(nn.Module):
    def __init__(self, d_model: int, freq_dim: int = 256) -> None:
        super().__init__()
        self.freq_dim = int(freq_dim)
        self.mlp = nn.Sequential(nn.Linear(2 * self.freq_dim, d_model), nn.SiLU(), nn.Linear(d_model, d_model))

    def _embed(self, t: torch.Tensor) -> torch.Tensor:
        half = self.freq_dim // 2
        freqs = torch.exp(-math.log(10_000) * torch.arange(half, dtype=torch.float32, device=t.device) / max(half, 1))
        args = 2.0 * math.pi * t[:, None].float() * freqs[None, :]
        return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)

    def forward(self, t_global: torch.Tensor, t_atomic: torch.Tensor) -> torch.Tensor:
        return self.mlp(torch.cat([self._embed(t_global), self._embed(t_atomic)], dim=-1))


def _masked_mean(coords: torch.Tensor, pad_mask: torch.Tensor) -> torch.Tensor:
    valid = (~pad_mask).to(coords.dtype)
    return (coords * valid[..., None]).sum(1, keepdim=True) / valid.sum(1, keepdim=True).clamp_min(1.0)[..., None]


def recenter_coordinates(coords: torch.Tensor, pad_mask: torch.Tensor) -> torch.Tensor:
    coords = coords.masked_fill(pad_mask[..., None], 0.0)
    return (coords - _masked_mean(coords, pad_mask)).masked_fill(pad_mask[..., None], 0.0)


class EDMModel(nn.Module):
    """Atom/coordinate denoiser: token projection -> trunk -> atom head + equivariant pair head.

    Mirrors ``QM9EDMModel(use_geometry_bias=False, coord_embed_mode="none", coord_head_mode="equivariant")``
    with the default noise conditioning (sigma channel concatenated to the atom features and adaLN).
    """

    def __init__(self, *, atom_channels: int = 6, d_model: int = 512, n_heads: int = 8, n_layers: int = 12,
                 attn_types: Optional[Sequence[str]] = None, mlp_ratio: float = 4.0, simplicial_impl: str = "auto",
                 simplicial_precision: str = "bf16_tc", pair_hidden_dim: int = 128, pair_n_rbf: int = 16,
                 pair_rbf_max: float = 4.0) -> None:  # fmt: skip
        super().__init__()
        if attn_types is None:  # layers alternate MHA and 2-simplicial attention
            attn_types = ["mha" if i % 2 == 0 else "simplicial" for i in range(n_layers)]
        self.atom_channels = int(atom_channels)
        self.atom_proj = nn.Linear(self.atom_channels + 1, d_model)
        self.conditioning = TimeEmbedder(d_model)
        self.trunk = TransformerTrunk(d_model, n_heads, attn_types, mlp_ratio=mlp_ratio,
                                      simplicial_impl=simplicial_impl, simplicial_precision=simplicial_precision)  # fmt: skip
        self.atom_head = nn.Sequential(nn.LayerNorm(d_model), nn.Linear(d_model, d_model), nn.SiLU(),
                                       nn.Linear(d_model, atom_channels))  # fmt: skip
        self.pair_head = nn.Sequential(nn.Linear(2 * d_model + pair_n_rbf, pair_hidden_dim), nn.SiLU(),
                                       nn.Linear(pair_hidden_dim, 1))  # fmt: skip
        nn.init.zeros_(self.pair_head[-1].weight)
        nn.init.zeros_(self.pair_head[-1].bias)
        self.register_buffer("_pair_rbf_centers", torch.linspace(0.0, pair_rbf_max, pair_n_rbf), persistent=False)
        delta = pair_rbf_max / max(pair_n_rbf - 1, 1)
        self.register_buffer("_pair_rbf_gamma", torch.tensor(1.0 / max(delta * delta, 1e-6)), persistent=False)
        self._pair_rbf_gamma_value = float(torch.tensor(1.0 / max(delta * delta, 1e-6), dtype=torch.float32))

    def _coord_delta(self, trunk_out: torch.Tensor, coords: torch.Tensor, pad_mask: torch.Tensor) -> torch.Tensor:
        d = trunk_out.shape[-1]
        w0, b0 = self.pair_head[0].weight, self.pair_head[0].bias
        kernel_fits = trunk_out.is_cuda and trunk_out.dtype in (torch.float32, torch.bfloat16)
        if kernel_fits and tuple(w0[:, 2 * d :].shape) == (fused.PAIR_HIDDEN, fused.PAIR_RBF) and not coords.requires_grad:
            # per-atom halves of the first Linear (two GEMMs), everything per pair in one kernel
            a = F.linear(trunk_out, w0[:, :d])
            b = F.linear(trunk_out, w0[:, d : 2 * d], b0)
            return fused.equivariant_pair_head(a, b, coords, ~pad_mask, w0[:, 2 * d :], self.pair_head[2].weight,
                                               self.pair_head[2].bias, self._pair_rbf_centers, self._pair_rbf_gamma_value)  # fmt: skip
        return self._coord_delta_torch(trunk_out, coords, pad_mask)

    def _coord_delta_torch(self, trunk_out: torch.Tensor, coords: torch.Tensor, pad_mask: torch.Tensor) -> torch.Tensor:
        # non-periodic pair geometry (geometry/adapters.py:83-125): deltas, distances, RMS-radius normalisation
        coords = coords.float()
        valid = ~pad_mask
        pair_mask = valid[:, :, None] & valid[:, None, :]
        delta = coords[:, :, None, :] - coords[:, None, :, :]
        dist = delta.square().sum(-1).clamp_min(0.0).sqrt()
        sq = coords.square().sum(-1) * valid
        rms = (sq.sum(1) / valid.sum(1).clamp_min(1)).clamp_min(1e-8).sqrt()
        dist_norm = (dist / rms[:, None, None].clamp_min(1e-8)) * pair_mask
        delta = delta * pair_mask[..., None]
        rbf = torch.exp(-self._pair_rbf_gamma * (dist_norm[..., None] - self._pair_rbf_centers.view(1, 1, 1, -1)).square())
        # pair_head[0] applied to cat[h_i, h_j, rbf_ij] (models/qm9.py:478-486), evaluated as
        # W_i h_i + W_j h_j + W_r rbf_ij + b so the (B,N,N,2d+16) concatenation is never materialised
        d = trunk_out.shape[-1]
        w0, b0 = self.pair_head[0].weight, self.pair_head[0].bias
        hid = (F.linear(trunk_out, w0[:, :d])[:, :, None, :] + F.linear(trunk_out, w0[:, d : 2 * d])[:, None, :, :]
               + F.linear(rbf.to(trunk_out.dtype), w0[:, 2 * d :], b0))  # fmt: skip
        w = self.pair_head[2](self.pair_head[1](hid)).squeeze(-1)
        w = w.masked_fill(~pair_mask, 0.0)
        w = w - torch.diag_embed(torch.diagonal(w, dim1=-2, dim2=-1))
        out = (w[..., None] * delta).sum(dim=2) / valid.sum(1, keepdim=True).clamp_min(1.0)[..., None]
        out = out.masked_fill(pad_mask[..., None], 0.0)
        return (out - _masked_mean(out, pad_mask)).masked_fill(pad_mask[..., None], 0.0)

    def forward(self, atom_noisy, coords_noisy, pad_mask, sigma, lattice=None):
        if sigma.ndim == 2:
            sigma = sigma[:, 0]
        sigma_cond = torch.log(sigma.clamp_min(1e-8)) / 4.0
        feat = sigma_cond[:, None, None].expand(-1, atom_noisy.shape[1], 1).masked_fill(pad_mask[..., None], 0.0)
        tokens = self.atom_proj(torch.cat([atom_noisy, feat], dim=-1))
        cond = self.conditioning(sigma_cond, sigma_cond)
        trunk_out = self.trunk(tokens, cond, pad_mask=pad_mask)
        atom_delta = self.atom_head[1:](layer_norm(trunk_out, self.atom_head[0])).masked_fill(pad_mask[..., None], 0.0)
        return atom_delta, self._coord_delta(trunk_out, coords_noisy, pad_mask)


class EDMPreconditioner(nn.Module):
    """EDM input/output scaling around the denoiser (tasks/edm.py:34-81)."""

    def __init__(self, model: nn.Module, *, sigma_data: float = 0.5) -> None:
        super().__init__()
        self.model = model
        self.sigma_data = float(sigma_data)

    def forward(self, atom_noisy, coords_noisy, pad_mask, sigma, *, lattice=None):
        if sigma.ndim == 2:
            sigma = sigma[:, 0]
        sigma = sigma.float()
        sd2 = self.sigma_data**2
        c_skip = sd2 / (sigma.square() + sd2)
        c_out = sigma * self.sigma_data / torch.sqrt(sigma.square() + sd2)
        c_in = 1.0 / torch.sqrt(sd2 + sigma.square())
        atom_in = atom_noisy * c_in[:, None, None]
        coords_in = recenter_coordinates(coords_noisy * c_in[:, None, None], pad_mask)
        atom_delta, coord_delta = self.model(atom_in, coords_in, pad_mask, sigma, lattice=lattice)
        atom_clean = atom_in - atom_delta
        coord_clean = recenter_coordinates(coords_in - coord_delta, pad_mask)
        atom_den = (c_skip[:, None, None] * atom_noisy + c_out[:, None, None] * atom_clean).masked_fill(pad_mask[..., None], 0.0)
        coord_den = recenter_coordinates(c_skip[:, None, None] * coords_noisy + c_out[:, None, None] * coord_clean, pad_mask)
        return atom_den, coord_den


def _masked_sample_mse(pred: torch.Tensor, target: torch.Tensor, pad_mask: torch.Tensor) -> torch.Tensor:
    # summed over atoms and channels, divided by the number of real atoms (tasks/edm.py:19-31)
    valid = (~pad_mask)[..., None].to(pred.dtype)
    err = (pred - target).square() * valid
    dims = tuple(range(1, err.ndim))
    return err.sum(dims) / valid.sum(dims).clamp_min(1.0)


class EDMLoss:
    """Noise sampling + weighted masked MSE of one denoising step (tasks/edm.py:84-150).

    ``sigma`` / ``atom_noise`` / ``coord_noise`` may be supplied so that two implementations can be compared on
    identical draws; otherwise they come from the global RNG exactly where the reference draws them.
    """

    def __init__(self, *, p_mean: float = -1.2, p_std: float = 1.2, sigma_data: float = 0.5,
                 atom_feature_scale: float = 4.0, charge_feature_scale: float = 8.0, num_atom_types: int = 5,
                 max_weight: Optional[float] = 1000.0) -> None:  # fmt: skip
        self.p_mean, self.p_std, self.sigma_data = float(p_mean), float(p_std), float(sigma_data)
        self.atom_feature_scale, self.charge_feature_scale = float(atom_feature_scale), float(charge_feature_scale)
        self.num_atom_types = int(num_atom_types)
        self.max_weight = max_weight

    def clean_features(self, atom_types, pad_mask, charges=None):
        onehot = F.one_hot(atom_types.clamp(0, self.num_atom_types - 1), self.num_atom_types).float()
        onehot = onehot.masked_fill(pad_mask[..., None], 0.0) / self.atom_feature_scale
        ch = torch.zeros_like(atom_types) if charges is None else charges
        ch = ch.masked_fill(pad_mask, 0).float()[..., None] / self.charge_feature_scale
        return torch.cat([onehot, ch], dim=-1)

    def __call__(self, net: EDMPreconditioner, atom_types, coords, pad_mask, *, charges=None, sigma=None,
                 atom_noise=None, coord_noise=None):  # fmt: skip
        atom_clean = self.clean_features(atom_types, pad_mask, charges)
        coords_clean = recenter_coordinates(coords.float(), pad_mask)
        if sigma is None:
            sigma = torch.exp(torch.randn(atom_clean.shape[0], device=atom_clean.device) * self.p_std + self.p_mean)
        weight = (sigma.square() + self.sigma_data**2) / (sigma * self.sigma_data).square()
        if self.max_weight is not None:
            weight = weight.clamp(max=self.max_weight)
        if atom_noise is None:
            atom_noise = torch.randn_like(atom_clean)
        if coord_noise is None:
            coord_noise = torch.randn_like(coords_clean)
        atom_noisy = atom_clean + atom_noise * sigma[:, None, None]
        cn = recenter_coordinates(coord_noise * sigma[:, None, None], pad_mask)
        coords_noisy = recenter_coordinates(coords_clean + cn, pad_mask)
        atom_den, coords_den = net(atom_noisy, coords_noisy, pad_mask, sigma)
        atom_loss = _masked_sample_mse(atom_den, atom_clean, pad_mask)
        coord_loss = _masked_sample_mse(coords_den, coords_clean, pad_mask)
        loss = (weight * atom_loss).mean() + (weight * coord_loss).mean()
        return loss, {"sigma": sigma, "atom_loss": atom_loss, "coord_loss": coord_loss, "loss_weight": weight}
