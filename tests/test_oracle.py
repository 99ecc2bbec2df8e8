"""The CPU oracles against the golden vectors the reference produced (tests/golden/make_golden.py)."""
import pytest
import torch

from oracle import geom_ref, sparse_ref
from oracle.simplicial_ref import SimplicialInputs, simplicial_forward, simplicial_forward_backward


def _inputs(g, *, bias=False):
    valid = g["valid"].bool()
    kw = dict(q=g["in_q"], k1=g["in_k1"], v1=g["in_v1"], k2=g["in_k2"], v2=g["in_v2"], query_valid=valid,
              pair_key_valid=valid, pair_valid=g["pair_valid"].bool() if "pair_valid" in g else None)  # fmt: skip
    if bias:
        for k in ("u", "v_bias", "w", "gate", "angle_left", "angle_right", "angle_gate", "message_left",
                  "message_right", "message_basis"):  # fmt: skip
            if "in_" + k in g:
                kw[k] = g["in_" + k]
    return SimplicialInputs(**kw)


@pytest.mark.parametrize("name,bias", [("pad", False), ("holes", False), ("bias", True), ("factorized", True), ("factorized_tiles", True), ("peaked", False), ("config1", False)])
def test_simplicial_oracle_matches_reference(golden, name, bias):
    g = golden(f"simplicial_{name}.npz")
    inp = _inputs(g, bias=bias)
    out, grads = simplicial_forward_backward(inp, g["grad_out"])
    torch.testing.assert_close(out, g["out"], atol=2e-6, rtol=1e-5)
    for k, gr in grads.items():
        torch.testing.assert_close(gr, g["d_" + k], atol=5e-6, rtol=1e-4, msg=lambda m, k=k: f"d_{k}: {m}")


def test_simplicial_oracle_zero_rows(golden):
    """Invalid queries give exact zeros; padded rows get exactly zero gradients."""
    g = golden("simplicial_pad.npz")
    inp = _inputs(g)
    out, grads = simplicial_forward_backward(inp, g["grad_out"])
    pad = ~g["valid"].bool()
    assert out[pad[:, None, :].expand(-1, out.shape[1], -1)].abs().max() == 0
    for k in ("q", "k1", "v1", "k2", "v2"):
        assert grads[k][pad[:, None, :].expand(-1, out.shape[1], -1)].abs().max() == 0


def test_simplicial_known_answer(golden):
    """Single visible pair (0,0) -> out = v1_0 * v2_0 = [3, 10] (reference tests/test_simplicial_attention.py:448-463)."""
    g = golden("simplicial_known_answer.npz")
    ones = torch.ones(1, 2, dtype=torch.bool)
    inp = SimplicialInputs(q=g["q"], k1=g["k1"], v1=g["v1"], k2=g["k2"], v2=g["v2"], query_valid=ones,
                           pair_key_valid=ones, pair_valid=g["pair_valid"].bool())  # fmt: skip
    out, lse = simplicial_forward(inp, return_lse=True)
    torch.testing.assert_close(out, g["out"])
    torch.testing.assert_close(out[0, 0], torch.tensor([[3.0, 10.0], [3.0, 10.0]]))
    torch.testing.assert_close(lse, torch.zeros_like(lse))  # one pair with logit 0


def test_simplicial_bf16_modes(golden):
    g = golden("simplicial_bf16.npz")
    valid = g["valid"].bool()
    inp = SimplicialInputs(**{k: g["in_" + k].bfloat16() for k in ("q", "k1", "v1", "k2", "v2")}, query_valid=valid,
                           pair_key_valid=valid)  # fmt: skip
    out32 = simplicial_forward(inp, fp32_core=True)
    # the reference casts its fp32-core result back to bf16 (simplicial_attention.py:344)
    torch.testing.assert_close(out32.bfloat16().float(), g["out_fp32_core"], atol=1e-7, rtol=1e-2)
    out_native = simplicial_forward(inp, fp32_core=False).float()
    # bf16 result: identical up to the last bf16 bit
    torch.testing.assert_close(out_native, g["out_native"], atol=2e-5, rtol=1e-2)


def test_lse_is_logsumexp_of_visible_logits(golden):
    g = golden("simplicial_holes.npz")
    inp = _inputs(g)
    _, lse = simplicial_forward(inp, return_lse=True)
    q, k1, k2 = inp.q, inp.k1, inp.k2
    logits = torch.einsum("bhid,bhjd,bhkd->bhijk", q, k1, k2)
    kv = inp.pair_key_valid
    m = (kv[:, :, None] & kv[:, None, :] & inp.pair_valid)[:, None, None]
    ref = torch.logsumexp(logits.masked_fill(~m, float("-inf")).flatten(-2), -1)
    ref = torch.where(inp.query_valid[:, None, :] & m.flatten(-2).any(-1), ref, torch.zeros_like(ref))
    torch.testing.assert_close(lse, ref, atol=1e-5, rtol=1e-5)


# ---- geometry -------------------------------------------------------------------------------


def test_min_image_known_answer(golden):
    """frac 0.1 vs 0.9 in a unit cube -> distance 0.2 (reference tests/test_geometry.py:30-39)."""
    g = golden("geometry_known_answer.npz")
    d2 = sparse_ref.periodic_pair_dist2(g["frac"], g["lattice"])
    torch.testing.assert_close(d2.sqrt(), g["pair_dist"], atol=1e-6, rtol=1e-6)
    cell = sparse_ref.lattice_to_cell(g["lattice"])
    dc = geom_ref.pair_dist2(g["frac"][0], cell[0]).sqrt()
    assert abs(dc[0, 1].item() - 0.2) < 1e-6 and dc[0, 0].item() == 0.0


def test_periodic_distances_match_reference(golden):
    g = golden("geometry.npz")
    n = g["num_atoms"]
    N = g["frac"].shape[1]
    valid = torch.arange(N)[None, :] < n[:, None]
    pm = valid[:, :, None] & valid[:, None, :]
    d2 = sparse_ref.periodic_pair_dist2(g["frac"], g["lattice"]) * pm
    torch.testing.assert_close(d2, g["pair_dist2"], atol=1e-5, rtol=1e-5)
    cell = sparse_ref.lattice_to_cell(g["lattice"])
    dc = torch.stack([geom_ref.pair_dist2(g["frac"][b], cell[b]) for b in range(2)]) * pm
    # fixed-order fp32 formula vs the reference's einsum: a few ulp apart at most
    torch.testing.assert_close(dc, g["pair_dist2"], atol=2e-5, rtol=2e-6)


def test_knn_oracle_matches_reference_sort(golden):
    g = golden("geometry.npz")
    cell = sparse_ref.lattice_to_cell(g["lattice"])
    idx, d2 = geom_ref.knn_topk(g["frac"], cell, g["num_atoms"], int(g["knn_k"]))
    ref = g["knn_idx"]
    mism = idx != ref
    if mism.any():  # only near ties may flip between the two fp32 evaluation orders
        dref = sparse_ref.periodic_pair_dist2(g["frac"], g["lattice"])
        b, i, t = torch.nonzero(mism, as_tuple=True)
        a = dref[b, i, idx[b, i, t].long()]
        c = dref[b, i, ref[b, i, t].long()]
        assert torch.allclose(a, c, rtol=1e-5, atol=1e-6)
    assert mism.float().mean() < 0.01
    # and the torch restatement of the selection agrees with the C one on the C distances
    dc = torch.stack([geom_ref.pair_dist2(g["frac"][b], cell[b]) for b in range(2)])
    idx2, _ = sparse_ref.knn_from_dist2(dc, g["num_atoms"], int(g["knn_k"]))
    assert torch.equal(idx2, idx)


def test_knn_ties_and_edge_cases():
    # a simple cubic lattice of points: every atom has 6 equidistant neighbours -> pure tie-breaking
    # (spacing 1/4 is exact in binary, so the six distances really are bit-equal)
    pts = torch.tensor([[i, j, k] for i in range(4) for j in range(4) for k in range(4)], dtype=torch.float32) / 4.0
    cell = torch.eye(3)[None] * 4.0
    idx, d2 = geom_ref.knn_topk(pts[None], cell, torch.tensor([64]), 6)
    dall = geom_ref.pair_dist2(pts, cell[0])
    ref_idx, _ = sparse_ref.knn_from_dist2(dall[None], torch.tensor([64]), 6)
    assert torch.equal(idx, ref_idx)
    assert torch.allclose(d2, torch.ones_like(d2))
    # ascending index among ties
    assert (idx[0, :, 1:] > idx[0, :, :-1]).all()
    # fewer atoms than k, empty structure, single atom
    idx, d2 = geom_ref.knn_topk(pts[None, :4], cell, torch.tensor([3]), 8)
    assert (idx[0, :3, 2:] == -1).all() and (idx[0, 3] == -1).all() and torch.isinf(d2[0, 3]).all()
    idx, _ = geom_ref.knn_topk(pts[None, :4], cell, torch.tensor([0]), 4)
    assert (idx == -1).all()
    idx, d2 = geom_ref.knn_topk(pts[None, :1], cell, torch.tensor([1]), 2, include_self=True)
    assert idx[0, 0, 0] == 0 and idx[0, 0, 1] == -1 and d2[0, 0, 0] == 0


def test_blocklist_oracle_properties():
    g = torch.Generator().manual_seed(3)
    from matterformer_b200.sparse import cell_grid_dims
    from matterformer_b200.synthetic import random_triclinic_lattices

    lat = random_triclinic_lattices(2, g, 8.0, 14.0)
    frac = torch.rand(2, 100, 3, generator=g) * 3 - 1  # also outside [0,1)
    n = torch.tensor([100, 70])
    cell = sparse_ref.lattice_to_cell(lat)
    gd = cell_grid_dims(cell, 3.0)
    perm, count, cols, mask = geom_ref.cell_sort_blocklist(frac, cell, n, gd, 3.0)
    T = 4
    for b in range(2):
        nb = int(n[b])
        p = perm[b].long()
        assert sorted(p[:nb].tolist()) == list(range(nb)) and p[nb:].tolist() == list(range(nb, 100))
        d = geom_ref.pair_dist2(frac[b], cell[b]).sqrt()
        vis = d[p][:, p] <= 3.0
        vis[nb:, :] = False
        vis[:, nb:] = False
        vis = torch.nn.functional.pad(vis, (0, 128 - 100, 0, 128 - 100))
        bits = ((mask[b].long()[..., None] >> torch.arange(32)) & 1).bool()  # (T,T,32,32)
        dense = bits.permute(0, 2, 1, 3).reshape(128, 128)
        assert torch.equal(dense, vis)
        active = vis.view(T, 32, T, 32).any(3).any(1)
        for i in range(T):
            want = torch.nonzero(active[i]).flatten().tolist()
            assert count[b, i] == len(want) and cols[b, i, : len(want)].tolist() == want
            assert (cols[b, i, len(want) :] == -1).all()


def test_masked_attention_matches_reference(golden):
    g = golden("geometry.npz")
    n = g["num_atoms"]
    N = g["frac"].shape[1]
    valid = (torch.arange(N)[None, :] < n[:, None])[:, None, :, None]
    for kind in ("radius", "local"):
        q, k, v = (g[x].clone().requires_grad_(True) for x in ("q", "k", "v"))
        if kind == "radius":
            vis = sparse_ref.radius_visible(g["frac"], g["lattice"], n, float(g["cutoff"]))
        else:
            vis = sparse_ref.band_visible(N, n, int(g["window"]))
        out = sparse_ref.masked_attention(q, k, v, vis) * valid
        dq, dk, dv = torch.autograd.grad(out, [q, k, v], g["grad_out"] * valid)
        torch.testing.assert_close(out, g[f"{kind}_out"], atol=1e-5, rtol=1e-5)
        for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
            torch.testing.assert_close(t, g[f"{kind}_{name}"], atol=1e-5, rtol=1e-4)


def test_pair_head_oracle_matches_reference(golden):
    """The restated coordinate head against outputs and gradients of the reference model's own method."""
    from oracle.pair_head_ref import equivariant_coord_delta, rbf_constants

    g = golden("pair_head.npz")
    centers, gamma = rbf_constants()
    torch.testing.assert_close(centers, g["centers"], atol=0, rtol=0)
    assert float(gamma) == float(g["gamma"])
    leaves = [g[n].clone().requires_grad_(True) for n in ("trunk_out", "w0", "b0", "w1", "b1")]
    out = equivariant_coord_delta(leaves[0], g["coords"], g["pad_mask"].bool(), *leaves[1:], centers, gamma)
    torch.testing.assert_close(out, g["out"], atol=1e-5, rtol=1e-5)
    grads = torch.autograd.grad(out, leaves, g["grad_out"])
    for n, gr in zip(("trunk_out", "w0", "b0", "w1", "b1"), grads):
        torch.testing.assert_close(gr, g["d_" + n], atol=1e-4, rtol=1e-4, msg=lambda m, n=n: f"d{n}: {m}")
    pad = g["pad_mask"].bool()
    assert out[pad].abs().max() == 0
    assert out[2].abs().max() == 0 and out[3].abs().max() == 0  # one atom, no atoms: nothing to move
