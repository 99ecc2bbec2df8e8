"""Parity of the periodic kNN, block list, radius block-sparse and local-window attention kernels
(through the C ABI): integer outputs bit-exact against the fixed-order C oracle, attention within
1e-4 (fp32) / 2e-2 (bf16) of the masked-SDPA oracle and of the reference's golden vectors."""
import pytest
import torch

import matterformer_b200 as mfb
from matterformer_b200 import synthetic
from matterformer_b200.sparse import cell_grid_dims
from oracle import geom_ref, sparse_ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _cells(B, N, seed, lo=8.0, hi=14.0):
    g = torch.Generator().manual_seed(seed)
    lat = synthetic.random_triclinic_lattices(B, g, lo, hi)
    frac = torch.rand(B, N, 3, generator=g)
    return lat, frac, g


def test_knn_matches_reference_golden(golden):
    g = golden("geometry.npz")
    cell = sparse_ref.lattice_to_cell(g["lattice"])
    idx, d2 = mfb.knn_topk(g["frac"].to(DEV), cell.to(DEV), g["num_atoms"].to(DEV), k=int(g["knn_k"]))
    oi, od = geom_ref.knn_topk(g["frac"], cell, g["num_atoms"], int(g["knn_k"]))
    assert torch.equal(idx.cpu(), oi)
    assert torch.equal(d2.cpu()[oi >= 0], od[oi >= 0])  # bit-exact distances
    assert (idx.cpu() != g["knn_idx"]).float().mean() < 0.01  # vs the reference's einsum order: near ties only


@pytest.mark.parametrize("B,N,k,include_self", [(3, 200, 16, False), (2, 77, 8, True), (1, 1, 4, False), (2, 300, 32, False)])
def test_knn_bit_exact_vs_oracle(B, N, k, include_self):
    lat, frac, g = _cells(B, N, seed=N + k)
    frac = frac * 2.5 - 0.7  # coordinates outside [0,1) too
    cell = sparse_ref.lattice_to_cell(lat)
    n = torch.randint(max(1, N // 2), N + 1, (B,), generator=g)
    n[0] = N
    idx, d2 = mfb.knn_topk(frac.to(DEV), cell.to(DEV), n.to(DEV), k=k, include_self=include_self)
    oi, od = geom_ref.knn_topk(frac, cell, n, k, include_self)
    assert torch.equal(idx.cpu(), oi)
    fin = oi >= 0
    assert torch.equal(d2.cpu()[fin], od[fin]) and torch.isinf(d2.cpu()[~fin]).all()


@pytest.mark.parametrize("B,N,k,lo,hi", [(4, 600, 16, 8.0, 14.0), (2, 1500, 8, 20.0, 30.0), (3, 40, 32, 5.0, 7.0),
                                         (2, 900, 16, 4.0, 40.0)])
def test_knn_cell_list_bit_exact(B, N, k, lo, hi):
    """Wrapped coordinates (the cell-list search proper, incl. strongly anisotropic cells): same bits as the
    all-pairs kernel and as the oracle."""
    lat, frac, g = _cells(B, N, seed=7 * N + k, lo=lo, hi=hi)
    cell = sparse_ref.lattice_to_cell(lat)
    n = torch.randint(max(1, N // 3), N + 1, (B,), generator=g)
    n[0] = N
    args = (frac.to(DEV), cell.to(DEV), n.to(DEV))
    ic, dc = mfb.knn_topk(*args, k=k, method="cells")
    ip, dp = mfb.knn_topk(*args, k=k, method="pairs")
    assert torch.equal(ic, ip) and torch.equal(dc, dp)
    geom_ref.set_threads(geom_ref.default_threads())
    oi, od = geom_ref.knn_topk(frac, cell, n, k)
    assert torch.equal(ic.cpu(), oi)
    fin = oi >= 0
    assert torch.equal(dc.cpu()[fin], od[fin])


def test_knn_ties_go_to_lower_index():
    pts = torch.tensor([[i, j, k] for i in range(4) for j in range(4) for k in range(4)], dtype=torch.float32) / 4.0
    cell = torch.eye(3)[None] * 4.0
    idx, d2 = mfb.knn_topk(pts[None].to(DEV), cell.to(DEV), torch.tensor([64]).to(DEV), k=6)
    oi, _ = geom_ref.knn_topk(pts[None], cell, torch.tensor([64]), 6)
    assert torch.equal(idx.cpu(), oi)
    assert (idx[0, :, 1:] > idx[0, :, :-1]).all() and torch.equal(d2.cpu(), torch.ones(1, 64, 6))


def test_knn_config4_slice_and_properties():
    """Full size (B=32, N=4096, k=16): two cells bit-exact against the oracle, all cells sorted and self-free."""
    t = synthetic.config4(with_qkv=False)
    cell = sparse_ref.lattice_to_cell(t["lattice"])
    idx, d2 = mfb.knn_topk(t["pos"].to(DEV), cell.to(DEV), t["num_atoms"].to(DEV), k=16)
    idx, d2 = idx.cpu(), d2.cpu()
    geom_ref.set_threads(geom_ref.default_threads())
    oi, od = geom_ref.knn_topk(t["pos"][:2], cell[:2], t["num_atoms"][:2], 16)
    assert torch.equal(idx[:2], oi) and torch.equal(d2[:2], od)
    assert (d2[..., 1:] >= d2[..., :-1]).all()
    assert (idx != torch.arange(4096)[None, :, None]).all() and (idx >= 0).all() and (idx < 4096).all()
    # a checksum that any two bit-identical runs share
    idx2, _ = mfb.knn_topk(t["pos"].to(DEV), cell.to(DEV), t["num_atoms"].to(DEV), k=16)
    assert torch.equal(idx2.cpu(), idx)


@pytest.mark.parametrize("B,N,cutoff", [(2, 100, 3.0), (3, 257, 4.0), (1, 31, 2.0), (1, 32, 50.0)])
def test_blocklist_bit_exact_vs_oracle(B, N, cutoff):
    lat, frac, g = _cells(B, N, seed=N)
    frac = frac * 3 - 1
    cell = sparse_ref.lattice_to_cell(lat)
    n = torch.randint(max(1, N // 2), N + 1, (B,), generator=g)
    gd = cell_grid_dims(cell, cutoff)
    blocks = mfb.build_radius_blocks(frac.to(DEV), cell.to(DEV), n.to(DEV), cutoff, grid_dims=gd)
    perm, count, cols, mask = geom_ref.cell_sort_blocklist(frac, cell, n, gd, cutoff)
    assert torch.equal(blocks.perm.cpu(), perm)
    assert torch.equal(blocks.block_count.cpu(), count)
    assert torch.equal(blocks.block_cols.cpu(), cols)
    assert torch.equal(blocks.block_mask.cpu(), mask)
    inv = blocks.inverse_perm.cpu().long()
    assert torch.equal(torch.gather(perm.long(), 1, inv), torch.arange(N)[None].expand(B, -1))


def _attn_ref(q, k, v, go, vis, valid):
    q, k, v = (x.clone().float().requires_grad_(True) for x in (q, k, v))
    out = sparse_ref.masked_attention(q, k, v, vis) * valid
    dq, dk, dv = torch.autograd.grad(out, [q, k, v], go.float() * valid)
    return out.detach(), dq, dk, dv


def _check(got, ref, tol, what):
    # relative to the largest reference value; the floor keeps all-zero references (a token that only
    # sees itself has dq = dk = 0 up to fp32 summation order) from demanding exact zeros
    scale = max(ref.abs().max().item(), 1.0 if tol < 1e-3 else 1e-2)
    err = (got.float().cpu() - ref).abs().max().item()
    assert err <= tol * scale, f"{what}: {err:.3e} vs scale {scale:.3e}"


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("D", [32, 64, 128])
def test_radius_attention_vs_oracle(dtype, tol, D):
    B, H, N, cutoff = 2, 2, 150, 3.5
    lat, frac, g = _cells(B, N, seed=D)
    n = torch.tensor([150, 97])
    cell = sparse_ref.lattice_to_cell(lat)
    q, k, v, go = (torch.randn(B, H, N, D, generator=g).to(dtype) for _ in range(4))
    valid = (torch.arange(N)[None, :] < n[:, None])[:, None, :, None]
    vis = sparse_ref.radius_visible(frac, lat, n, cutoff)
    ref = _attn_ref(q.float(), k.float(), v.float(), go.float(), vis, valid)
    blocks = mfb.build_radius_blocks(frac.to(DEV), cell.to(DEV), n.to(DEV), cutoff)
    qd, kd, vd = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
    out = mfb.radius_block_sparse_attention(qd, kd, vd, blocks, sorted_inputs=False)
    grads = torch.autograd.grad(out, [qd, kd, vd], go.to(DEV))
    for got, want, what in zip((out.detach(), *grads), ref, ("out", "dq", "dk", "dv")):
        _check(got, want, tol, what)
    assert out.detach()[~valid.expand_as(out).to(DEV)].abs().max() == 0


def test_radius_attention_matches_reference_golden(golden):
    g = golden("geometry.npz")
    cell = sparse_ref.lattice_to_cell(g["lattice"])
    blocks = mfb.build_radius_blocks(g["frac"].to(DEV), cell.to(DEV), g["num_atoms"].to(DEV), float(g["cutoff"]))
    q, k, v = (g[x].to(DEV).requires_grad_(True) for x in ("q", "k", "v"))
    out = mfb.radius_block_sparse_attention(q, k, v, blocks, sorted_inputs=False)
    dq, dk, dv = torch.autograd.grad(out, [q, k, v], g["grad_out"].to(DEV))
    for got, name in ((out.detach(), "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        torch.testing.assert_close(got.cpu(), g[f"radius_{name}"], atol=1e-4, rtol=1e-4)
    ql, kl, vl = (g[x].to(DEV).requires_grad_(True) for x in ("q", "k", "v"))
    out = mfb.local_window_attention(ql, kl, vl, g["num_atoms"].to(DEV), window=int(g["window"]))
    dq, dk, dv = torch.autograd.grad(out, [ql, kl, vl], g["grad_out"].to(DEV))
    for got, name in ((out.detach(), "out"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        torch.testing.assert_close(got.cpu(), g[f"local_{name}"], atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("N,window", [(200, 64), (50, 64), (97, 8), (1, 2)])
def test_local_attention_vs_oracle(dtype, tol, N, window):
    B, H, D = 2, 2, 64
    g = torch.Generator().manual_seed(N + window)
    n = torch.tensor([N, max(1, N - 13)])
    q, k, v, go = (torch.randn(B, H, N, D, generator=g).to(dtype) for _ in range(4))
    valid = (torch.arange(N)[None, :] < n[:, None])[:, None, :, None]
    vis = sparse_ref.band_visible(N, n, window)
    ref = _attn_ref(q.float(), k.float(), v.float(), go.float(), vis, valid)
    qd, kd, vd = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
    out = mfb.local_window_attention(qd, kd, vd, n.to(DEV), window=window)
    grads = torch.autograd.grad(out, [qd, kd, vd], go.to(DEV))
    for got, want, what in zip((out.detach(), *grads), ref, ("out", "dq", "dk", "dv")):
        _check(got, want, tol, what)


def test_sparse_deterministic_and_empty():
    B, H, N, D = 1, 2, 96, 64
    g = torch.Generator().manual_seed(1)
    q, k, v, go = (torch.randn(B, H, N, D, generator=g).bfloat16().to(DEV) for _ in range(4))
    n = torch.tensor([96]).to(DEV)

    def run():
        qq, kk, vv = (x.clone().requires_grad_(True) for x in (q, k, v))
        o = mfb.local_window_attention(qq, kk, vv, n, window=32)
        return (o.detach(), *torch.autograd.grad(o, [qq, kk, vv], go))

    a, b = run(), run()
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    o = mfb.local_window_attention(q, k, v, torch.tensor([0]).to(DEV), window=32)
    assert o.abs().max() == 0


def test_radius_attention_at_benchmark_size():
    """One cell of the benchmark's crystals (N = 1024, triclinic 15-30 A, 0.9 A minimum separation, cutoff 6 A;
    two heads to keep the CPU oracle affordable): a row tile then walks most of the 32 column tiles, which is the
    path the benchmark times.  Block list bit for bit against the C oracle; forward and the three gradients against
    dense masked attention at 2e-2 (bf16)."""
    from matterformer_b200 import synthetic

    t = synthetic.config3(seed=0, batch=1, n=1024, heads=2)
    frac, lat, n, cutoff = t["pos"], t["lattice"], t["num_atoms"], t["cutoff"]
    cell = sparse_ref.lattice_to_cell(lat)
    gd = cell_grid_dims(cell, cutoff)
    blocks = mfb.build_radius_blocks(frac.to(DEV), cell.to(DEV), n.to(DEV), cutoff, grid_dims=gd)
    perm, count, cols, mask = geom_ref.cell_sort_blocklist(frac, cell, n, gd, cutoff)
    assert torch.equal(blocks.perm.cpu(), perm)
    assert torch.equal(blocks.block_count.cpu(), count)
    assert torch.equal(blocks.block_cols.cpu(), cols)
    assert torch.equal(blocks.block_mask.cpu(), mask)
    assert count.float().mean() > 16, "the benchmark's cells are dense: most column tiles are active"
    q, k, v, go = t["q"], t["k"], t["v"], t["grad_out"]
    valid = torch.ones(1, 1, 1024, 1, dtype=torch.bool)
    vis = sparse_ref.radius_visible(frac, lat, n, cutoff)
    ref = _attn_ref(q.float(), k.float(), v.float(), go.float(), vis, valid)
    qd, kd, vd = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
    out = mfb.radius_block_sparse_attention(qd, kd, vd, blocks, sorted_inputs=False)
    grads = torch.autograd.grad(out, [qd, kd, vd], go.to(DEV))
    for got, want, what in zip((out.detach(), *grads), ref, ("out", "dq", "dk", "dv")):
        _check(got, want, 2e-2, what)


def test_local_attention_at_benchmark_size():
    """One cell of the benchmark's local-window workload (N = 4096 tokens, window 64, two heads), forward and the
    three gradients against dense attention with the band as additive mask."""
    from matterformer_b200 import synthetic

    t = synthetic.config4(seed=0, batch=1, n=4096, heads=2)
    q, k, v, go, n = t["q"], t["k_"], t["v"], t["grad_out"], t["num_atoms"]
    valid = torch.ones(1, 1, 4096, 1, dtype=torch.bool)
    vis = sparse_ref.band_visible(4096, n, 64)
    ref = _attn_ref(q.float(), k.float(), v.float(), go.float(), vis, valid)
    qd, kd, vd = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
    out = mfb.local_window_attention(qd, kd, vd, n.to(DEV), window=64)
    grads = torch.autograd.grad(out, [qd, kd, vd], go.to(DEV))
    for got, want, what in zip((out.detach(), *grads), ref, ("out", "dq", "dk", "dv")):
        _check(got, want, 2e-2, what)


@pytest.fixture
def tcgen05_sparse():
    prev = mfb.set_sparse_backend("tcgen05")
    yield
    mfb.set_sparse_backend(prev)
    assert mfb.sparse_device_status() == 0, "a bounded device-side wait expired"


@pytest.mark.parametrize("N,n_list,cutoff", [(152, [152, 97], 3.5), (128, [128, 1], 3.5), (260, [260, 129], 3.0),
                                             (64, [64, 33], 4.0), (200, [0, 200], 3.5)])  # fmt: skip
def test_radius_attention_tcgen05_vs_oracle(tcgen05_sparse, N, n_list, cutoff):
    """The 128-row tcgen05 tiles on short structures: ragged last tiles, a padded second structure, an empty one."""
    B, H, D = 2, 2, 64
    lat, frac, g = _cells(B, N, seed=N)
    n = torch.tensor(n_list)
    cell = sparse_ref.lattice_to_cell(lat)
    q, k, v, go = (torch.randn(B, H, N, D, generator=g).bfloat16() for _ in range(4))
    valid = (torch.arange(N)[None, :] < n[:, None])[:, None, :, None]
    vis = sparse_ref.radius_visible(frac, lat, n, cutoff)
    ref = _attn_ref(q.float(), k.float(), v.float(), go.float(), vis, valid)
    blocks = mfb.build_radius_blocks(frac.to(DEV), cell.to(DEV), n.to(DEV), cutoff)
    qd, kd, vd = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
    out = mfb.radius_block_sparse_attention(qd, kd, vd, blocks, sorted_inputs=False)
    grads = torch.autograd.grad(out, [qd, kd, vd], go.to(DEV))
    for got, want, what in zip((out.detach(), *grads), ref, ("out", "dq", "dk", "dv")):
        _check(got, want, 2e-2, what)
    assert out.detach()[~valid.expand_as(out).to(DEV)].abs().max() == 0


def test_radius_attention_tcgen05_ignores_what_padding_holds(tcgen05_sparse):
    """Padded tokens may hold anything, NaN included: nothing of it may reach the real atoms' results."""
    B, H, N, D, cutoff = 1, 2, 160, 64, 3.5
    lat, frac, g = _cells(B, N, seed=3)
    n = torch.tensor([100])
    cell = sparse_ref.lattice_to_cell(lat)
    q, k, v, go = (torch.randn(B, H, N, D, generator=g).bfloat16() for _ in range(4))
    blocks = mfb.build_radius_blocks(frac.to(DEV), cell.to(DEV), n.to(DEV), cutoff)

    def run(fill):
        ts = []
        for x in (q, k, v, go):
            x = x.clone()
            x[:, :, 100:] = fill
            ts.append(x.to(DEV))
        qd, kd, vd = (x.requires_grad_(True) for x in ts[:3])
        # sorted order: the first 100 rows are the real atoms
        out = mfb.radius_block_sparse_attention(qd, kd, vd, blocks, sorted_inputs=True)
        return (out.detach(), *torch.autograd.grad(out, [qd, kd, vd], ts[3]))

    clean, dirty = run(0.0), run(float("nan"))
    for a, b in zip(clean, dirty):
        assert torch.equal(a[:, :, :100], b[:, :, :100])
        assert b[:, :, 100:].abs().max() == 0


@pytest.mark.parametrize("N,window", [(200, 64), (300, 8), (128, 64), (516, 128)])
def test_local_attention_tcgen05_vs_oracle(tcgen05_sparse, N, window):
    B, H, D = 2, 2, 64
    g = torch.Generator().manual_seed(N + window)
    n = torch.tensor([N, max(1, N - 77)])
    q, k, v, go = (torch.randn(B, H, N, D, generator=g).bfloat16() for _ in range(4))
    valid = (torch.arange(N)[None, :] < n[:, None])[:, None, :, None]
    vis = sparse_ref.band_visible(N, n, window)
    ref = _attn_ref(q.float(), k.float(), v.float(), go.float(), vis, valid)
    qd, kd, vd = (x.to(DEV).requires_grad_(True) for x in (q, k, v))
    out = mfb.local_window_attention(qd, kd, vd, n.to(DEV), window=window)
    grads = torch.autograd.grad(out, [qd, kd, vd], go.to(DEV))
    for got, want, what in zip((out.detach(), *grads), ref, ("out", "dq", "dk", "dv")):
        _check(got, want, 2e-2, what)


def test_sparse_tcgen05_is_reproducible_and_matches_the_warp_level_tiles(tcgen05_sparse):
    from matterformer_b200 import synthetic

    t = synthetic.config3(seed=1, batch=1, n=512, heads=2)
    cell = sparse_ref.lattice_to_cell(t["lattice"])
    blocks = mfb.build_radius_blocks(t["pos"].to(DEV), cell.to(DEV), t["num_atoms"].to(DEV), t["cutoff"])

    def run():
        qd, kd, vd = (t[x].to(DEV).requires_grad_(True) for x in ("q", "k", "v"))
        out = mfb.radius_block_sparse_attention(qd, kd, vd, blocks, sorted_inputs=False)
        return (out.detach(), *torch.autograd.grad(out, [qd, kd, vd], t["grad_out"].to(DEV)))

    a, b = run(), run()
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    prev = mfb.set_sparse_backend("mma")
    try:
        c = run()
    finally:
        mfb.set_sparse_backend(prev)
    for x, y, what in zip(a, c, ("out", "dq", "dk", "dv")):
        _check(x, y.float().cpu(), 2e-2, what)


def test_tcgen05_path_works_on_a_thread_that_has_not_touched_the_device(tcgen05_sparse):
    """The tensor-map encoder needs a context bound to the calling thread; a thread that was only handed cached device
    memory (the backward thread of the autograd engine after a warm-up) has none.  The library binds one itself."""
    import threading

    from matterformer_b200 import synthetic

    t = synthetic.config3(seed=2, batch=1, n=256, heads=2)
    cell = sparse_ref.lattice_to_cell(t["lattice"])
    blocks = mfb.build_radius_blocks(t["pos"].to(DEV), cell.to(DEV), t["num_atoms"].to(DEV), t["cutoff"])
    q, k, v = (t[x].to(DEV) for x in ("q", "k", "v"))
    want = mfb.radius_block_sparse_attention(q, k, v, blocks)  # warms the allocator: the thread below gets cached blocks
    torch.cuda.synchronize()
    box = {}

    def work():
        try:
            box["out"] = mfb.radius_block_sparse_attention(q, k, v, blocks)
            torch.cuda.synchronize()
        except Exception as exc:  # noqa: BLE001 - reported by the assertion below
            box["error"] = exc

    del want
    th = threading.Thread(target=work)
    th.start()
    th.join()
    assert "error" not in box, box.get("error")
    assert torch.equal(box["out"], mfb.radius_block_sparse_attention(q, k, v, blocks))


@pytest.mark.parametrize("B,H,N,D,window", [(3, 8, 29, 64, 64), (2, 4, 100, 32, 16), (2, 2, 7, 128, 64)])
def test_local_attention_on_the_packed_projection(B, H, N, D, window):
    """q, k, v read inside the (B,N,3,H,D) projection, out written as (B,N,H*D): bit for bit the head-major call."""
    g = torch.Generator().manual_seed(B + N)
    qkv = torch.randn(B, N, 3 * H * D, generator=g).bfloat16().to(DEV)
    go = torch.randn(B, N, H * D, generator=g).bfloat16().to(DEV)
    n = torch.randint(1, N + 1, (B,), generator=g).to(DEV)
    from matterformer_b200.sparse import local_window_attention_packed

    x = qkv.clone().requires_grad_(True)
    out = local_window_attention_packed(x, H, n, window=window)
    (gx,) = torch.autograd.grad(out, [x], go)
    parts = [qkv.view(B, N, 3, H, D)[:, :, i].transpose(1, 2).contiguous().requires_grad_(True) for i in range(3)]
    prev = mfb.set_sparse_backend("mma")
    try:
        y = mfb.local_window_attention(*parts, n, window=window)
        grads = torch.autograd.grad(y, parts, go.view(B, N, H, D).transpose(1, 2).contiguous())
    finally:
        mfb.set_sparse_backend(prev)
    assert torch.equal(out.view(B, N, H, D).transpose(1, 2), y)
    assert torch.equal(gx.view(B, N, 3, H, D), torch.stack([t.transpose(1, 2) for t in grads], dim=2))
