"""CPU baselines taken from the reference itself (TEST / BENCHMARK INFRASTRUCTURE, never imported by the product).

When the reference package has been installed next to the repository (``python -m pip install --no-index
--no-build-isolation --no-deps --target baseline/_ref <reference checkout>``; the directory is not part of the
source tree) these helpers run the reference's own torch code on the host cores, so that ``bench.py`` can quote
``cpu_baseline.kind = "reference"``.  Without it every helper reports unavailability and the callers fall back to
the restatements in ``oracle/``.

What is called, by path inside the reference project:
* ``simplicial_attention_torch_from_projected`` (src/matterformer/models/simplicial_attention.py:206-344),
* ``PeriodicGeometryAdapter`` (src/matterformer/geometry/adapters.py:127-212),
* ``QM9EDMModel`` / ``AdaLNBlock`` / ``EDMPreconditioner`` / ``EDMLoss``
  (src/matterformer/models/qm9.py, models/transformer.py, tasks/edm.py).
"""
from __future__ import annotations

import sys
from pathlib import Path
from types import SimpleNamespace

import torch

REF_DIR = Path(__file__).resolve().parents[1] / "baseline" / "_ref"
NAMES = ("q", "k1", "v1", "k2", "v2")


def available() -> bool:
    return (REF_DIR / "matterformer" / "models" / "simplicial_attention.py").is_file()


def _import(name: str):
    import importlib

    if not available():
        raise RuntimeError(f"the reference is not installed under {REF_DIR}")
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    return importlib.import_module(name)


def simplicial_forward_backward(tensors: dict, valid: torch.Tensor, grad_out: torch.Tensor, chunk_size: int = 16):
    """Forward + backward of the reference's dense torch path (fp32, autograd) on padded molecules."""
    sa = _import("matterformer.models.simplicial_attention")
    x = [tensors[n].float().requires_grad_(True) for n in NAMES]
    B, _, N, _ = x[0].shape
    mask = sa.SimplicialAttentionMask.from_key_padding_mask(~valid, batch_size=B, num_tokens=N, device=x[0].device)
    out = sa.simplicial_attention_torch_from_projected(*x, attention_mask=mask, chunk_size=chunk_size)
    grads = torch.autograd.grad(out, x, grad_out.float())
    return out.detach(), dict(zip(NAMES, grads))


def periodic_masked_attention(frac, lattice, q, k, v, cutoff: float, grad_out=None):
    """Radius attention as the reference would compute it: adapter distances -> additive 0 / finfo.min mask ->
    scaled_dot_product_attention (regular_attention.py:251-268).  Returns (out, grads or None)."""
    ad = _import("matterformer.geometry.adapters")
    adapter = ad.PeriodicGeometryAdapter(pbc_radius=1, lattice_repr="y1")
    dist = adapter(frac, lattice=lattice).pair_dist
    q, k, v = (t.float().requires_grad_(grad_out is not None) for t in (q, k, v))
    bias = torch.zeros_like(dist).masked_fill(dist > cutoff, torch.finfo(torch.float32).min)
    out = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=bias[:, None])
    if grad_out is None:
        return out, None
    return out.detach(), torch.autograd.grad(out, (q, k, v), grad_out.float())


def periodic_pair_dist2(frac, lattice):
    ad = _import("matterformer.geometry.adapters")
    return ad.PeriodicGeometryAdapter(pbc_radius=1, lattice_repr="y1")(frac, lattice=lattice).pair_dist2


def build_edm_net(d_model: int = 512, n_heads: int = 8, n_layers: int = 12, seed: int = 0):
    """The benchmark trunk assembled from the reference's own blocks: simplicial trunk with the even blocks
    replaced by MHA blocks, geometry bias off, torch simplicial path."""
    qm9 = _import("matterformer.models.qm9")
    tr = _import("matterformer.models.transformer")
    edm = _import("matterformer.tasks.edm")
    torch.manual_seed(seed)
    model = qm9.QM9EDMModel(d_model=d_model, n_heads=n_heads, n_layers=n_layers, attn_type="simplicial",
                            use_geometry_bias=False, simplicial_impl="torch")  # fmt: skip
    for i in range(0, n_layers, 2):
        model.trunk.blocks[i] = tr.AdaLNBlock(d_model=d_model, n_heads=n_heads, attn_type="mha")
    return edm.EDMPreconditioner(model, sigma_data=1.0), edm.EDMLoss(sigma_data=1.0)


def edm_step(net, loss_fn, batch: dict, optimizer=None) -> float:
    """One EDM denoising step (forward, backward, optional optimizer step) of the reference model in fp32."""
    types, pad = batch["atom_types"], batch["pad_mask"]
    ns = SimpleNamespace(
        coords=batch["coords"], pad_mask=pad, lattice=None,
        atom_onehot=lambda: torch.nn.functional.one_hot(types, 5).float().masked_fill(pad[..., None], 0.0),
        formal_charges=lambda: torch.zeros_like(types),
    )  # fmt: skip
    if optimizer is not None:
        optimizer.zero_grad(set_to_none=True)
    loss, _ = loss_fn(net, ns)
    loss.backward()
    if optimizer is not None:
        optimizer.step()
    return float(loss.detach())
