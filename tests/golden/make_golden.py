"""Generates the golden vectors under tests/golden/ by running the REFERENCE implementation.

Run in a container that has the reference checked out:

    PYTHONPATH=<reference>/src python tests/golden/make_golden.py

It imports ``matterformer`` (the reference package) and writes small ``.npz`` files next to this
script.  The parity tests load those files; nothing at test time needs the reference itself.
Every case is seeded; rerunning reproduces the files bit for bit on the same torch build.
"""
from __future__ import annotations

import math
import sys
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

try:
    from matterformer.geometry.adapters import PeriodicGeometryAdapter
    from matterformer.models.simplicial_attention import (
        SimplicialAttentionMask,
        SimplicialFactorizedBias,
        SimplicialLowRankAngleResidual,
        SimplicialLowRankMessageResidual,
        simplicial_attention_torch_from_projected,
    )
except ImportError as exc:  # pragma: no cover
    sys.exit(f"the reference package is not importable ({exc}); set PYTHONPATH to <reference>/src")

OUT = Path(__file__).resolve().parent
torch.set_num_threads(8)


def _np(t):
    return t.detach().cpu().float().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def simplicial_case(name, B, H, N, D, *, seed, n_valid=None, holes=False, bias=False, scale=1.0, keep=None,
                    bf16_values=False):
    """``bf16_values``: every operand is rounded to bf16 first (and kept in fp32), so that a bf16 kernel sees exactly
    the values the reference computed with."""
    g = torch.Generator().manual_seed(seed)

    def leaf(x):
        return (x.bfloat16().float() if bf16_values else x).requires_grad_(True)

    t = {k: leaf(torch.randn(B, H, N, D, generator=g) * scale) for k in ("q", "k1", "v1", "k2", "v2")}
    grad_out = torch.randn(B, H, N, D, generator=g)
    if bf16_values:
        grad_out = grad_out.bfloat16().float()
    if n_valid is None:
        n_valid = [N] * B
    valid = torch.arange(N)[None, :] < torch.tensor(n_valid)[:, None]
    pair_valid = None
    if holes:
        pair_valid = torch.rand(B, N, N, generator=g) > 0.3
    mask = SimplicialAttentionMask(query_valid=valid, pair_key_valid=valid, pair_valid=pair_valid)
    extra = {}
    kwargs = {}
    if bias:
        R, Rm = 5, 3
        for k in ("u", "v_bias", "w"):
            extra[k] = leaf(torch.randn(B, H, N, N, generator=g) * 0.5)
        extra["gate"] = leaf(torch.randn(B, H, N, generator=g))
        kwargs = dict(
            factorized_bias=SimplicialFactorizedBias(u=extra["u"], v=extra["v_bias"], w=extra["w"], gate=extra["gate"])
        )
    if bias is True:  # bias == "factorized" stops at u, v, w, gate
        extra["angle_left"] = torch.randn(B, H, N, N, R, generator=g).requires_grad_(True)
        extra["angle_right"] = torch.randn(B, H, N, N, R, generator=g).requires_grad_(True)
        extra["angle_gate"] = torch.randn(B, H, N, generator=g).requires_grad_(True)
        extra["message_left"] = torch.randn(B, H, N, N, Rm, generator=g).requires_grad_(True)
        extra["message_right"] = torch.randn(B, H, N, N, Rm, generator=g).requires_grad_(True)
        extra["message_basis"] = (torch.randn(H, Rm, D, generator=g) / math.sqrt(D)).requires_grad_(True)
        kwargs = dict(
            factorized_bias=SimplicialFactorizedBias(u=extra["u"], v=extra["v_bias"], w=extra["w"], gate=extra["gate"]),
            angle_residual=SimplicialLowRankAngleResidual(
                left=extra["angle_left"], right=extra["angle_right"], gate=extra["angle_gate"]
            ),
            message_residual=SimplicialLowRankMessageResidual(left=extra["message_left"], right=extra["message_right"]),
            message_basis=extra["message_basis"],
        )
    out = simplicial_attention_torch_from_projected(
        t["q"], t["k1"], t["v1"], t["k2"], t["v2"], attention_mask=mask, chunk_size=3, **kwargs
    )
    leaves = {**t, **extra}
    grads = torch.autograd.grad(out, list(leaves.values()), grad_out, allow_unused=True)
    sl = slice(None) if keep is None else slice(0, keep)
    arrays = {"grad_out": _np(grad_out[sl]), "valid": _np(valid[sl]), "out": _np(out[sl])}
    if pair_valid is not None:
        arrays["pair_valid"] = _np(pair_valid[sl])
    for (k, v), gr in zip(leaves.items(), grads):
        if k == "message_basis":
            arrays["in_" + k] = _np(v)
            arrays["d_" + k] = _np(gr)
        else:
            arrays["in_" + k] = _np(v[sl])
            arrays["d_" + k] = _np(gr[sl])
    np.savez_compressed(OUT / f"simplicial_{name}.npz", **arrays)
    print("wrote", name, {k: a.shape for k, a in arrays.items() if k in ("out",)})


def known_answer():
    """Single visible pair (0,0): the output is v1_0 * v2_0 (reference tests/test_simplicial_attention.py:448-463)."""
    q = torch.zeros(1, 1, 2, 2)
    k1 = torch.zeros(1, 1, 2, 2)
    k2 = torch.zeros(1, 1, 2, 2)
    v1 = torch.tensor([[[[1.0, 2.0], [100.0, 200.0]]]])
    v2 = torch.tensor([[[[3.0, 5.0], [300.0, 500.0]]]])
    pair_valid = torch.zeros(1, 2, 2, dtype=torch.bool)
    pair_valid[0, 0, 0] = True
    mask = SimplicialAttentionMask(
        query_valid=torch.ones(1, 2, dtype=torch.bool), pair_key_valid=torch.ones(1, 2, dtype=torch.bool), pair_valid=pair_valid
    )
    out = simplicial_attention_torch_from_projected(q, k1, v1, k2, v2, attention_mask=mask)
    np.savez_compressed(OUT / "simplicial_known_answer.npz", q=_np(q), k1=_np(k1), v1=_np(v1), k2=_np(k2), v2=_np(v2),
                        pair_valid=_np(pair_valid), out=_np(out))  # fmt: skip
    print("known answer out", out.flatten().tolist())


def bf16_case():
    """The reference's default (same-dtype) path on bf16 inputs: logits rounded to bf16 before the softmax."""
    g = torch.Generator().manual_seed(21)
    B, H, N, D = 1, 2, 40, 64
    t = {k: (torch.randn(B, H, N, D, generator=g) / 8.0).bfloat16() for k in ("q", "k1", "v1", "k2", "v2")}
    valid = torch.arange(N)[None, :] < torch.tensor([33])[:, None]
    mask = SimplicialAttentionMask(query_valid=valid, pair_key_valid=valid)
    out_native = simplicial_attention_torch_from_projected(t["q"], t["k1"], t["v1"], t["k2"], t["v2"], attention_mask=mask)
    out_fp32 = simplicial_attention_torch_from_projected(
        t["q"], t["k1"], t["v1"], t["k2"], t["v2"], attention_mask=mask, fp32_core=True
    )
    arrays = {"in_" + k: _np(v) for k, v in t.items()}
    arrays.update(valid=_np(valid), out_native=_np(out_native), out_fp32_core=_np(out_fp32))
    np.savez_compressed(OUT / "simplicial_bf16.npz", **arrays)
    print("bf16 case native-vs-fp32core max diff", (out_native.float() - out_fp32.float()).abs().max().item())


def triclinic(g, B):
    lat = torch.empty(B, 6)
    for b in range(B):
        lengths = 6.0 + 6.0 * torch.rand(3, generator=g)
        ang = torch.deg2rad(70.0 + 40.0 * torch.rand(3, generator=g))
        lat[b, :3] = torch.log(lengths)
        lat[b, 3:] = torch.cos(ang)
    return lat


def geometry_cases():
    g = torch.Generator().manual_seed(5)
    B, N = 2, 48
    lat = triclinic(g, B)
    frac = torch.rand(B, N, 3, generator=g)
    num_atoms = torch.tensor([48, 37])
    pad = torch.arange(N)[None, :] >= num_atoms[:, None]
    adapter = PeriodicGeometryAdapter(pbc_radius=1, lattice_repr="y1")
    feats = adapter(frac, pad_mask=pad, lattice=lat)
    d2 = feats.pair_dist2
    # kNN by stable sort of the reference's distances (self excluded, ties -> lower index)
    k = 8
    d = d2.clone().masked_fill(pad[:, None, :], float("inf"))
    d = d + torch.diag_embed(torch.full((B, N), float("inf")))
    val, idx = torch.sort(d, dim=-1, stable=True)
    idx = idx[..., :k].to(torch.int32)
    idx = torch.where(pad[:, :, None], torch.full_like(idx, -1), idx)
    # masked attention through SDPA exactly like RotaryMultiheadAttention.forward's core call
    H, D = 2, 32
    q, kk, v = (torch.randn(B, H, N, D, generator=g) for _ in range(3))
    grad_out = torch.randn(B, H, N, D, generator=g)
    q.requires_grad_(True), kk.requires_grad_(True), v.requires_grad_(True)
    cutoff = 4.0
    valid = ~pad
    visible = (feats.pair_dist <= cutoff) & valid[:, :, None] & valid[:, None, :]
    bias = torch.zeros(B, N, N).masked_fill(~visible, torch.finfo(torch.float32).min)
    out = F.scaled_dot_product_attention(q, kk, v, attn_mask=bias[:, None])
    out = out * valid[:, None, :, None]
    dq, dk, dv = torch.autograd.grad(out, [q, kk, v], grad_out * valid[:, None, :, None])
    # band (local window) attention, window 16
    window = 16
    i = torch.arange(N)[:, None]
    j = torch.arange(N)[None, :]
    band = ((j >= i - window // 2) & (j <= i + window // 2 - 1))[None] & valid[:, :, None] & valid[:, None, :]
    bias_l = torch.zeros(B, N, N).masked_fill(~band, torch.finfo(torch.float32).min)
    out_l = F.scaled_dot_product_attention(q, kk, v, attn_mask=bias_l[:, None]) * valid[:, None, :, None]
    dq_l, dk_l, dv_l = torch.autograd.grad(out_l, [q, kk, v], grad_out * valid[:, None, :, None])
    np.savez_compressed(
        OUT / "geometry.npz",
        lattice=_np(lat), frac=_np(frac), num_atoms=_np(num_atoms), pair_dist2=_np(d2), knn_idx=_np(idx), knn_k=k,
        q=_np(q), k=_np(kk), v=_np(v), grad_out=_np(grad_out), cutoff=cutoff,
        radius_out=_np(out), radius_dq=_np(dq), radius_dk=_np(dk), radius_dv=_np(dv),
        window=window, local_out=_np(out_l), local_dq=_np(dq_l), local_dk=_np(dk_l), local_dv=_np(dv_l),
    )  # fmt: skip
    # minimum-image known answer of the reference's tests/test_geometry.py:30-39
    frac2 = torch.tensor([[[0.1, 0.0, 0.0], [0.9, 0.0, 0.0]]])
    lat2 = torch.zeros(1, 6)
    f2 = adapter(frac2, pad_mask=None, lattice=lat2)
    np.savez_compressed(OUT / "geometry_known_answer.npz", frac=_np(frac2), lattice=_np(lat2), pair_dist=_np(f2.pair_dist))
    print("min-image known answer dist", f2.pair_dist[0, 0, 1].item())


def trunk_case():
    """EDM denoising step of an alternating MHA / simplicial trunk assembled from reference blocks (fp32, CPU)."""
    from types import SimpleNamespace

    from matterformer.models.qm9 import QM9EDMModel
    from matterformer.models.transformer import AdaLNBlock
    from matterformer.tasks.edm import EDMLoss, EDMPreconditioner, recenter_coordinates

    torch.manual_seed(123)
    d_model, heads, layers = 32, 2, 2
    model = QM9EDMModel(d_model=d_model, n_heads=heads, n_layers=layers, attn_type="simplicial", use_geometry_bias=False,
                        simplicial_impl="torch")  # fmt: skip
    for i in range(0, layers, 2):
        model.trunk.blocks[i] = AdaLNBlock(d_model=d_model, n_heads=heads, attn_type="mha")
    B, N = 3, 9
    n = torch.tensor([9, 6, 4])
    pad = torch.arange(N)[None, :] >= n[:, None]
    g = torch.Generator().manual_seed(7)
    atom_types = torch.randint(0, 5, (B, N), generator=g).masked_fill(pad, 0)
    coords = (torch.randn(B, N, 3, generator=g) * 1.5).masked_fill(pad[..., None], 0.0)
    net = EDMPreconditioner(model, sigma_data=1.0)
    with torch.no_grad():  # materialise the lazy layer, then move every parameter off its (partly zero) initial value
        net(torch.zeros(B, N, 6), recenter_coordinates(coords, pad), pad, torch.ones(B))
        pg = torch.Generator().manual_seed(9)
        for p in model.parameters():
            p.add_(torch.randn(p.shape, generator=pg) * 0.05)
    batch = SimpleNamespace(
        coords=coords, pad_mask=pad, lattice=None,
        atom_onehot=lambda: torch.nn.functional.one_hot(atom_types, 5).float().masked_fill(pad[..., None], 0.0),
        formal_charges=lambda: torch.zeros_like(atom_types),
    )  # fmt: skip
    loss_fn = EDMLoss(sigma_data=1.0)
    torch.manual_seed(2024)
    loss, diag = loss_fn(net, batch)
    # the same draws, in the order EDMLoss makes them (tasks/edm.py:118-130)
    torch.manual_seed(2024)
    z = torch.randn(B)
    sigma = torch.exp(z * loss_fn.p_std + loss_fn.p_mean)
    atom_noise = torch.randn(B, N, 6)
    coord_noise = torch.randn(B, N, 3)
    assert torch.equal(sigma, diag["sigma"])
    names = [k for k, _ in model.named_parameters()]
    grads = torch.autograd.grad(loss, list(model.parameters()))
    arrays = {"state/" + k: _np(v) for k, v in model.state_dict().items()}
    arrays.update({"grad/" + k: _np(gr) for k, gr in zip(names, grads)})
    arrays.update(atom_types=_np(atom_types), coords=_np(coords), pad_mask=_np(pad), sigma=_np(sigma),
                  atom_noise=_np(atom_noise), coord_noise=_np(coord_noise), loss=_np(loss.detach()),
                  atom_loss=_np(diag["atom_loss"].detach()), coord_loss=_np(diag["coord_loss"].detach()))  # fmt: skip
    np.savez_compressed(OUT / "trunk_edm.npz", **arrays)
    print("trunk case loss", float(loss), "params", sum(p.numel() for p in model.parameters()))


def sampler_case():
    """Stochastic Heun sampler of the reference (tasks/edm.py:153-233) on the trunk fixture's model: 5 steps, CPU."""
    from matterformer.models.qm9 import QM9EDMModel
    from matterformer.models.transformer import AdaLNBlock
    from matterformer.tasks.edm import EDMPreconditioner, edm_sampler

    g = np.load(OUT / "trunk_edm.npz")
    d_model, heads, layers = 32, 2, 2
    model = QM9EDMModel(d_model=d_model, n_heads=heads, n_layers=layers, attn_type="simplicial", use_geometry_bias=False,
                        simplicial_impl="torch")  # fmt: skip
    for i in range(0, layers, 2):
        model.trunk.blocks[i] = AdaLNBlock(d_model=d_model, n_heads=heads, attn_type="mha")
    net = EDMPreconditioner(model, sigma_data=1.0)
    with torch.no_grad():
        net(torch.zeros(3, 9, 6), torch.zeros(3, 9, 3), torch.zeros(3, 9, dtype=torch.bool), torch.ones(3))
    model.load_state_dict({k[len("state/"):]: torch.from_numpy(g[k]) for k in g.files if k.startswith("state/")})
    model.eval()
    num_atoms = torch.tensor([9, 6, 4])
    out = {}
    for name, kw in (("churn", dict(num_steps=5)), ("plain", dict(num_steps=3, s_churn=0.0, sigma_max=5.0))):
        torch.manual_seed(77)
        with torch.no_grad():
            atoms, coords, pad = edm_sampler(net, num_atoms, atom_channels=6, **kw)
        out[name + "_atoms"], out[name + "_coords"] = _np(atoms), _np(coords)
    np.savez_compressed(OUT / "sampler_edm.npz", num_atoms=_np(num_atoms), **out)
    print("sampler case", {k: v.shape for k, v in out.items()})


def batch_sampler_case():
    """Batches of the reference's GeomDrugsPaddedBatchSampler (data/geom_drugs.py:113-212) for a seeded list of atom
    counts: unshuffled, and shuffled with ``random.seed(5)``; stored flat with batch lengths."""
    import random

    from matterformer.data.geom_drugs import GeomDrugsPaddedBatchSampler

    g = torch.Generator().manual_seed(0)
    num_atoms = torch.randint(5, 182, (400,), generator=g)
    arrays = {"num_atoms": _np(num_atoms)}
    cases = {
        "caps": dict(max_examples_per_batch=16, max_padded_atoms_per_batch=1500, max_attention_cost_per_batch=150000),
        "drop": dict(max_examples_per_batch=8, max_attention_cost_per_batch=90000, drop_last=True),
    }
    for name, kw in cases.items():
        for shuffle in (False, True):
            random.seed(5)
            sampler = GeomDrugsPaddedBatchSampler(num_atoms, shuffle=shuffle, **kw)
            batches = list(sampler)
            key = f"{name}_{'shuffled' if shuffle else 'sorted'}"
            arrays[key + "_flat"] = np.asarray([i for b in batches for i in b], dtype=np.int64)
            arrays[key + "_sizes"] = np.asarray([len(b) for b in batches], dtype=np.int64)
            arrays[key + "_len"] = np.asarray(len(sampler), dtype=np.int64)
    np.savez_compressed(OUT / "batch_sampler.npz", **arrays)
    print("batch sampler cases", {k: v.shape for k, v in arrays.items() if k.endswith("sizes")})


def pair_head_case():
    """Equivariant coordinate head of the reference model on random trunk outputs: output and gradients (fp32, CPU)."""
    from matterformer.geometry.adapters import NonPeriodicGeometryAdapter
    from matterformer.models.qm9 import QM9EDMModel

    torch.manual_seed(31)
    d_model = 32
    model = QM9EDMModel(d_model=d_model, n_heads=2, n_layers=1, attn_type="mha", use_geometry_bias=False)
    g = torch.Generator().manual_seed(32)
    B, N = 4, 37
    with torch.no_grad():  # materialise the lazy first Linear; the second starts at zero: move every weight off its initial value
        model._equivariant_coord_delta(torch.zeros(1, 2, d_model), NonPeriodicGeometryAdapter()(torch.zeros(1, 2, 3)),
                                       torch.zeros(1, 2, dtype=torch.bool))  # fmt: skip
        for p in model.pair_head.parameters():
            p.add_(torch.randn(p.shape, generator=g) * 0.2)
    n = torch.tensor([37, 20, 1, 0])
    pad = torch.arange(N)[None, :] >= n[:, None]
    pad[1, 3] = True  # padding is usually a suffix; the head must not rely on it
    coords = (torch.randn(B, N, 3, generator=g) * 1.5).masked_fill(pad[..., None], 0.0)
    trunk_out = torch.randn(B, N, d_model, generator=g).requires_grad_(True)
    grad_out = torch.randn(B, N, 3, generator=g)
    geom = NonPeriodicGeometryAdapter()(coords, pad_mask=pad)
    out = model._equivariant_coord_delta(trunk_out, geom, pad)
    params = list(model.pair_head.parameters())
    grads = torch.autograd.grad(out, [trunk_out] + params, grad_out)
    arrays = dict(trunk_out=_np(trunk_out), coords=_np(coords), pad_mask=_np(pad), grad_out=_np(grad_out), out=_np(out),
                  w0=_np(params[0]), b0=_np(params[1]), w1=_np(params[2]), b1=_np(params[3]),
                  centers=_np(model._pair_rbf_centers), gamma=_np(model._pair_rbf_gamma),
                  d_trunk_out=_np(grads[0]), d_w0=_np(grads[1]), d_b0=_np(grads[2]), d_w1=_np(grads[3]), d_b1=_np(grads[4]))  # fmt: skip
    np.savez_compressed(OUT / "pair_head.npz", **arrays)
    print("pair head case", tuple(out.shape), float(out.abs().max()))


if __name__ == "__main__":
    if sys.argv[1:] == ["pair_head"]:  # regenerate this one fixture
        pair_head_case()
        sys.exit(0)
    if sys.argv[1:] == ["batch_sampler"]:  # regenerate this one fixture
        batch_sampler_case()
        sys.exit(0)
    if sys.argv[1:] == ["sampler"]:  # regenerate this one fixture (needs trunk_edm.npz)
        sampler_case()
        sys.exit(0)
    if sys.argv[1:] == ["factorized"]:  # regenerate this one fixture and leave the others as they are
        simplicial_case("factorized", 2, 2, 37, 16, seed=15, n_valid=[37, 20], holes=True, bias="factorized",
                        scale=0.5)  # fmt: skip
        sys.exit(0)
    if sys.argv[1:] == ["factorized_tiles"]:  # regenerate this one fixture
        simplicial_case("factorized_tiles", 3, 4, 29, 64, seed=16, n_valid=[29, 20, 11], holes=True, bias="factorized",
                        scale=0.5, bf16_values=True)  # fmt: skip
        sys.exit(0)
    trunk_case()
    simplicial_case("pad", 2, 4, 5, 8, seed=11, n_valid=[5, 3])
    simplicial_case("holes", 1, 2, 7, 8, seed=12, n_valid=[6], holes=True)
    simplicial_case("bias", 1, 2, 7, 8, seed=13, n_valid=[6], holes=True, bias=True)
    simplicial_case("peaked", 1, 2, 33, 16, seed=14, n_valid=[29], scale=1.5)
    simplicial_case("config1", 8, 8, 29, 32, seed=0, n_valid=[20, 12, 23, 18, 10, 18, 22, 19], scale=1 / math.sqrt(32), keep=2)
    simplicial_case("factorized", 2, 2, 37, 16, seed=15, n_valid=[37, 20], holes=True, bias="factorized", scale=0.5)
    simplicial_case("factorized_tiles", 3, 4, 29, 64, seed=16, n_valid=[29, 20, 11], holes=True, bias="factorized",
                    scale=0.5, bf16_values=True)  # fmt: skip
    sampler_case()
    batch_sampler_case()
    pair_head_case()
    known_answer()
    bf16_case()
    geometry_cases()
