"""Host-side plumbing checked on the CPU with fake kernels, the way the reference tests its own
autograd boundary (tests/test_simplicial_attention.py:713-814 monkeypatches the kernel entry points)."""
import pytest
import torch

import matterformer_b200.simplicial as S
from matterformer_b200.sparse import cell_grid_dims, lattice_latent_to_cell
from oracle import sparse_ref


def test_autograd_function_layout_with_fake_kernels(monkeypatch):
    calls = {}

    def fake_forward(q, k1, v1, k2, v2, **kw):
        calls["fwd"] = kw
        out = q + k1 + v1 + k2 + v2
        return out, torch.zeros(q.shape[:3]), out.float()

    def fake_backward(grad_out, q, k1, v1, k2, v2, out, lse, **kw):
        calls["bwd"] = kw
        g = grad_out
        return (g, 2 * g, 3 * g, 4 * g, 5 * g) + (None,) * 10

    monkeypatch.setattr(S, "cuda_simplicial_attention_forward", fake_forward)
    monkeypatch.setattr(S, "cuda_simplicial_attention_backward", fake_backward)
    t = [torch.randn(1, 2, 3, 4, requires_grad=True) for _ in range(5)]
    ok = torch.ones(1, 3, dtype=torch.bool)
    out = S.simplicial_attention_cuda(*t, query_valid=ok, pair_key_valid=ok, precision="ieee_fp32")
    assert calls["fwd"]["pair_valid"] is None and calls["fwd"]["u"] is None and calls["fwd"]["precision"] == "ieee_fp32"
    out.sum().backward()
    assert calls["bwd"]["pair_valid"] is None and calls["bwd"]["precision"] == "ieee_fp32"
    for i, x in enumerate(t):
        torch.testing.assert_close(x.grad, torch.full_like(x, float(i + 1)))
    # 21 inputs -> 21 gradients, None at the mask / flag slots
    pv = torch.ones(1, 3, 3, dtype=torch.bool)
    out = S.simplicial_attention_cuda(*t, query_valid=ok, pair_key_valid=ok, pair_valid=pv)
    assert calls["fwd"]["pair_valid"] is pv or torch.equal(calls["fwd"]["pair_valid"], pv)


def test_residual_operands_are_rejected_and_bias_is_checked():
    x = torch.zeros(1, 1, 2, 2)
    r = torch.zeros(1, 1, 2, 2, 3)
    assert S._angle_group(None, None, None, 1, 1, 2) is None
    with pytest.raises(ValueError, match="given together"):
        S._angle_group(r, None, None, 1, 1, 2)
    (al, ar, ag), rank = S._angle_group(r, r.double(), torch.zeros(1, 1, 2), 1, 1, 2)
    assert rank == 3 and ar.dtype == torch.float32
    with pytest.raises(RuntimeError, match="ranks up to 32"):
        S._angle_group(torch.zeros(1, 1, 2, 2, 40), torch.zeros(1, 1, 2, 2, 40), torch.zeros(1, 1, 2), 1, 1, 2)
    with pytest.raises(ValueError, match="message_basis must have shape"):
        S._message_group(r, r, torch.zeros(1, 2, 8), 1, 1, 2, 8)
    assert S._factorized_bias(None, None, None, None, 1, 1, 2) is None
    with pytest.raises(ValueError, match="given together"):
        S._factorized_bias(x, None, x, None, 1, 1, 2)
    with pytest.raises(ValueError, match="gate must have shape"):
        S._factorized_bias(x, x, x, x, 1, 1, 2)
    u, v, w, g = S._factorized_bias(x.half(), x, x, torch.zeros(1, 1, 2), 1, 1, 2)
    assert u.dtype == torch.float32 and g.shape == (1, 1, 2)


def test_backend_switch():
    prev = S.set_backend("generic")
    assert S.set_backend(prev) == "generic"
    with pytest.raises(ValueError):
        S.set_backend("triton")


def test_lattice_to_cell_matches_reference_restatement():
    g = torch.Generator().manual_seed(0)
    lat = torch.cat([torch.randn(5, 3, generator=g), torch.rand(5, 3, generator=g) * 0.6 - 0.3], -1)
    torch.testing.assert_close(lattice_latent_to_cell(lat), sparse_ref.lattice_to_cell(lat), atol=0, rtol=0)


def test_grid_dims():
    cell = torch.diag(torch.tensor([35.0, 12.0, 5.0]))[None]
    assert cell_grid_dims(cell, 6.0).tolist() == [[5, 2, 1]]
    # sheared cell: perpendicular width, not edge length
    cell = torch.tensor([[[10.0, 0, 0], [9.0, 4.0, 0], [0, 0, 10.0]]])
    assert cell_grid_dims(cell, 2.0).tolist() == [[2, 2, 5]]


def test_install_rebinds_reference_module():
    ref = pytest.importorskip("matterformer.models.simplicial_attention")
    saved = (ref.TRITON_AVAILABLE, ref.triton_simplicial_attention_forward, ref.triton_simplicial_attention_backward,
             ref.SimplicialAttention._triton_unavailable_reason)  # fmt: skip
    try:
        S.install(ref)
        assert ref.TRITON_AVAILABLE is True
        assert ref.triton_simplicial_attention_forward is S.cuda_simplicial_attention_forward
        attn = ref.SimplicialAttention(16, 2, impl="auto")
        out = attn(torch.randn(1, 3, 16))  # CPU tensors -> the reference's own torch path
        assert attn._last_impl_used == "torch" and out.shape == (1, 3, 16)
    finally:
        (ref.TRITON_AVAILABLE, ref.triton_simplicial_attention_forward, ref.triton_simplicial_attention_backward,
         ref.SimplicialAttention._triton_unavailable_reason) = saved  # fmt: skip


def test_attention_cost_batch_sampler_matches_reference_batches(golden):
    """Same batches as the reference's GeomDrugsPaddedBatchSampler (data/geom_drugs.py:113-212) for the same atom counts,
    caps and ``random`` seed -- fixture generated by the reference -- and the reference's own cap test
    (tests/test_geom_drugs_data.py:105-122)."""
    import random

    from matterformer_b200.batching import AttentionCostBatchSampler, simplicial_tile_steps

    g = golden("batch_sampler.npz")
    cases = {
        "caps": dict(max_examples_per_batch=16, max_padded_atoms_per_batch=1500, max_attention_cost_per_batch=150000),
        "drop": dict(max_examples_per_batch=8, max_attention_cost_per_batch=90000, drop_last=True),
    }
    for name, kw in cases.items():
        for shuffle in (False, True):
            key = f"{name}_{'shuffled' if shuffle else 'sorted'}"
            random.seed(5)
            sampler = AttentionCostBatchSampler(g["num_atoms"], shuffle=shuffle, **kw)
            batches = list(sampler)
            assert [len(b) for b in batches] == g[key + "_sizes"].tolist()
            assert [i for b in batches for i in b] == g[key + "_flat"].tolist()
            assert len(sampler) == int(g[key + "_len"])
    num_atoms = torch.tensor([12, 13, 14, 48, 49, 50])
    for batch in AttentionCostBatchSampler(num_atoms, max_examples_per_batch=4, max_padded_atoms_per_batch=100,
                                           max_attention_cost_per_batch=2500, shuffle=False):  # fmt: skip
        atoms = [int(num_atoms[i]) for i in batch]
        assert len(batch) <= 4 and max(atoms) * len(batch) <= 100 and max(atoms) ** 2 * len(batch) <= 2500
    # the added budget: work the row-packed kernels really do, not padded max^2 x batch
    s = AttentionCostBatchSampler(g["num_atoms"], max_examples_per_batch=64, max_tile_steps_per_batch=1500, shuffle=False)
    for batch in s:
        assert len(batch) == 1 or sum(simplicial_tile_steps(int(g["num_atoms"][i])) for i in batch) <= 1500
    with pytest.raises(ValueError, match="At least one batch budget"):
        AttentionCostBatchSampler(num_atoms, max_examples_per_batch=4)
