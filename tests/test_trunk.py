"""The trunk mirror against the reference's golden EDM step, and the data-parallel step on two CPU ranks."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from matterformer_b200.dp import build_edm_net, edm_train_step, shard_batch, wrap_data_parallel
from matterformer_b200.synthetic import config5_batch
from matterformer_b200.trunk import EDMLoss, EDMModel, EDMPreconditioner


def _golden_net(g, impl, precision="ieee_fp32", device="cpu"):
    model = EDMModel(d_model=32, n_heads=2, n_layers=2, simplicial_impl=impl, simplicial_precision=precision)
    state = {k[len("state/"):]: v for k, v in g.items() if k.startswith("state/")}
    model.load_state_dict(state, strict=True)  # the reference's own parameter names
    return EDMPreconditioner(model.to(device), sigma_data=1.0)


def _run_golden(g, impl, device, tol):
    net = _golden_net(g, impl, device=device)
    loss_fn = EDMLoss(sigma_data=1.0)
    loss, diag = loss_fn(net, g["atom_types"].to(device), g["coords"].to(device), g["pad_mask"].bool().to(device),
                         sigma=g["sigma"].to(device), atom_noise=g["atom_noise"].to(device),
                         coord_noise=g["coord_noise"].to(device))  # fmt: skip
    names = [k for k, _ in net.model.named_parameters()]
    grads = torch.autograd.grad(loss, list(net.model.parameters()))
    assert abs(float(loss) - float(g["loss"])) <= tol * max(1.0, abs(float(g["loss"])))
    torch.testing.assert_close(diag["atom_loss"].cpu(), g["atom_loss"], atol=tol, rtol=tol)
    torch.testing.assert_close(diag["coord_loss"].cpu(), g["coord_loss"], atol=tol, rtol=tol)
    for k, gr in zip(names, grads):
        ref = g["grad/" + k]
        scale = max(1.0, ref.abs().max().item())
        assert (gr.cpu() - ref).abs().max().item() <= 10 * tol * scale, k


def test_trunk_mirror_matches_reference_on_cpu(golden):
    _run_golden(golden("trunk_edm.npz"), "torch", "cpu", 1e-5)


@pytest.mark.parametrize("name,kw", [("churn", dict(num_steps=5)), ("plain", dict(num_steps=3, s_churn=0.0, sigma_max=5.0))])
def test_sampler_matches_reference_on_cpu(golden, name, kw):
    """Same seed, same draws in the same order: the samples of the reference's edm_sampler (tasks/edm.py:153-233)."""
    from matterformer_b200.sampler import edm_sample

    net = _golden_net(golden("trunk_edm.npz"), "torch")
    net.eval()
    g = golden("sampler_edm.npz")
    torch.manual_seed(77)
    atoms, coords, pad = edm_sample(net, g["num_atoms"].long(), atom_channels=6, **kw)
    torch.testing.assert_close(atoms, g[name + "_atoms"], atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(coords, g[name + "_coords"], atol=2e-5, rtol=1e-4)
    assert atoms[pad].abs().max() == 0 and coords[pad].abs().max() == 0


@pytest.mark.gpu
def test_sampler_graph_replay_equals_eager(golden):
    """On CUDA the denoiser is captured once and replayed for every noise level; the samples must not change."""
    from matterformer_b200.sampler import edm_sample

    net = _golden_net(golden("trunk_edm.npz"), "cuda", device="cuda:0")
    net.eval()
    n = torch.tensor([9, 6, 4, 1])
    outs = []
    for graph in (False, True):
        torch.manual_seed(5)
        outs.append(edm_sample(net, n, atom_channels=6, num_steps=6, use_cuda_graph=graph))
    torch.testing.assert_close(outs[0][0], outs[1][0], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(outs[0][1], outs[1][1], atol=1e-5, rtol=1e-5)
    assert torch.isfinite(outs[1][1]).all()


@pytest.mark.gpu
def test_trunk_with_cuda_kernels_matches_reference(golden):
    _run_golden(golden("trunk_edm.npz"), "cuda", "cuda:0", 1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("n_tokens,heads", [(29, 8), (32, 4), (7, 2)])
def test_mha_core_on_local_window_kernel_matches_torch(n_tokens, heads):
    """With at most 32 tokens the window-64 kernel is dense attention: same result as nn.MultiheadAttention
    at the real tokens, forward and parameter / input gradients (bf16 tolerance 2e-2 of the largest value)."""
    from matterformer_b200.trunk import RegularAttention

    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    d_model = 64 * heads
    ours = RegularAttention(d_model, heads).to(dev)
    ref = RegularAttention(d_model, heads, impl="torch").to(dev)
    ref.load_state_dict(ours.state_dict())
    B = 6
    n = torch.tensor([n_tokens, 1, max(1, n_tokens // 2), n_tokens, 3, n_tokens - 1]).clamp(min=1)
    pad = (torch.arange(n_tokens)[None, :] >= n[:, None]).to(dev)
    x0 = torch.randn(B, n_tokens, d_model, device=dev)
    go = torch.randn(B, n_tokens, d_model, device=dev) * (~pad)[..., None]
    res = []
    for mod in (ours, ref):
        x = x0.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y = mod(x, key_padding_mask=pad)
        grads = torch.autograd.grad(y.float(), [x, *mod.parameters()], go)
        res.append((y.float() * (~pad)[..., None], grads))
    assert ours._last_core_used == "cuda" and ref._last_core_used == "torch"
    (y1, g1), (y2, g2) = res
    assert (y1 - y2).abs().max() <= 2e-2 * y2.abs().max()
    for a, b in zip(g1, g2):
        assert (a.float() - b.float()).abs().max() <= 2e-2 * b.float().abs().max()


@pytest.mark.gpu
def test_mha_padding_with_holes_takes_the_torch_path():
    """The window kernel reads the padding as "the last N - n tokens".  A mask with a padded token in the middle is
    not of that form: the layer must notice and give nn.MultiheadAttention's answer, not attend to the hole."""
    from matterformer_b200.trunk import RegularAttention

    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    ours = RegularAttention(128, 2).to(dev)
    ref = RegularAttention(128, 2, impl="torch").to(dev)
    ref.load_state_dict(ours.state_dict())
    pad = torch.zeros(3, 12, dtype=torch.bool, device=dev)
    pad[0, 9:] = True  # a suffix
    pad[1, 4] = True  # a hole
    pad[2, 0] = True  # a padded first token
    x = torch.randn(3, 12, 128, device=dev)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y1 = ours(x, key_padding_mask=pad)
        y2 = ref(x, key_padding_mask=pad)
    assert ours._last_core_used == "torch"
    torch.testing.assert_close(y1, y2)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        ours(x, key_padding_mask=pad[:1].expand(3, -1).contiguous())
    assert ours._last_core_used == "cuda"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,N,C", [(5, 29, 512), (3, 1, 32), (2, 40, 1000), (1, 9, 8)])
def test_fused_adaln_passes_match_torch(B, N, C, dtype):
    """norm + modulate and the gated residual: outputs and every gradient against the chain of torch ops."""
    from matterformer_b200.fused import gated_residual, ln_modulate

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(B * 100 + N)
    x0 = (torch.randn(B, N, C, device=dev, generator=g) * 2 + 0.5).to(dtype)  # the residual stream in the same type
    shift0, scale0, gate0 = (torch.randn(B, C, device=dev, generator=g) for _ in range(3))
    a0 = torch.randn(B, N, C, device=dev, generator=g).to(dtype)
    go_h = torch.randn(B, N, C, device=dev, generator=g).to(dtype)
    go_y = torch.randn(B, N, C, device=dev, generator=g).to(dtype)
    tol = 1e-4 if dtype == torch.float32 else 2e-2

    def leaves():
        return [t.clone().requires_grad_(True) for t in (x0, shift0, scale0, gate0, a0)]

    n_real = torch.randint(0, N + 1, (B,), device=dev, generator=g)
    pad = torch.arange(N, device=dev)[None, :] >= n_real[:, None]
    for pad_mask in (None, pad):  # without, and with the padded rows cleared in the same pass
        x, shift, scale, gate, a = leaves()
        h = ln_modulate(x, shift, scale, eps=1e-6, out_dtype=dtype)
        y = gated_residual(x, gate, a, pad_mask)
        got = [h, y, *torch.autograd.grad([h, y], [x, shift, scale, gate, a], [go_h, go_y])]
        x, shift, scale, gate, a = leaves()
        h = (torch.nn.functional.layer_norm(x.float(), (C,), eps=1e-6) * (1 + scale[:, None]) + shift[:, None]).to(dtype)
        y = (x.float() + gate[:, None] * a.float()).to(dtype)
        if pad_mask is not None:
            y = y.masked_fill(pad_mask[..., None], 0.0)
        want = [h, y, *torch.autograd.grad([h, y], [x, shift, scale, gate, a], [go_h, go_y])]
        for name, p, q in zip(("h", "y", "dx", "dshift", "dscale", "dgate", "da"), got, want):
            err = (p.float() - q.float()).abs().max().item()
            assert err <= tol * max(1.0, q.float().abs().max().item()), f"{name} (pad {pad_mask is not None}): {err}"
        if pad_mask is not None:
            assert got[1][pad_mask].abs().max() == 0 if pad_mask.any() else True


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,N,G,H,D", [(3, 29, 5, 8, 64), (2, 7, 3, 2, 8), (1, 1, 1, 1, 128)])
def test_head_split_and_merge_match_torch(B, N, G, H, D, dtype):
    from matterformer_b200.fused import merge_heads, split_heads

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(N)
    packed0 = torch.randn(B, N, G * H * D, device=dev, generator=gen).to(dtype)
    scales = [0.125] + [1.0] * (G - 1)
    gos = [torch.randn(B, H, N, D, device=dev, generator=gen).to(dtype) for _ in range(G)]
    packed = packed0.clone().requires_grad_(True)
    outs = split_heads(packed, G, H, scales)
    merged = merge_heads(outs[0])
    used = [0] if G == 1 else [0, G - 1]  # the other groups get no gradient: their slots must come back as zeros
    (gp,) = torch.autograd.grad([outs[i] for i in used], [packed], [gos[i] for i in used])
    ref = packed0.clone().requires_grad_(True)
    parts = [ref.view(B, N, G, H, D)[:, :, g].transpose(1, 2) * scales[g] for g in range(G)]
    (gr,) = torch.autograd.grad([parts[i] for i in used], [ref], [gos[i] for i in used])
    for a, b2 in zip(outs, parts):
        assert torch.equal(a, b2.to(dtype).contiguous())
    assert torch.equal(merged, outs[0].transpose(1, 2).reshape(B, N, H * D))
    torch.testing.assert_close(gp.float(), gr.float(), atol=1e-6 if dtype == torch.float32 else 1e-2, rtol=1e-2)
    y = merged.detach().requires_grad_(True)
    x = outs[0].detach().clone().requires_grad_(True)
    (gx,) = torch.autograd.grad(merge_heads(x), [x], torch.ones_like(merged) * 2)
    assert torch.equal(gx, torch.full_like(x, 2))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("kind", ["radius", "local"])
def test_periodic_mha_layer_matches_dense_attention_with_the_adapter_mask(kind, dtype, tol):
    """The slot where a radius / local mask enters the reference's trunk is the additive ``(B*H, T, T)`` mask of the
    MHA layer (AdaLNBlock.forward, src/matterformer/models/transformer.py:254-268).  Same layer, same weights: the
    sparse kernels with a plan built from (frac, lattice) against ``nn.MultiheadAttention`` with the dense 0 / finfo.min
    mask made from the adapter's minimum-image distances (radius) or from the band over the cell-sorted order (local)."""
    from matterformer_b200.trunk import RegularAttention, plan_sparse_attention
    from oracle import sparse_ref

    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(5)
    B, N, H, C, cutoff = 2, 150, 2, 128, 3.5
    lat = torch.cat([torch.log(8.0 + 6.0 * torch.rand(B, 3, generator=g)), 0.4 * torch.rand(B, 3, generator=g) - 0.2], -1)
    frac = torch.rand(B, N, 3, generator=g)
    n = torch.tensor([150, 97])
    pad = torch.arange(N)[None, :] >= n[:, None]
    layer = RegularAttention(C, H).to(dev)
    x0 = torch.randn(B, N, C, generator=g)
    go = torch.randn(B, N, C, generator=g) * (~pad)[..., None]
    plan = plan_sparse_attention(frac.to(dev), lat.to(dev), pad.to(dev), cutoff, kind=kind, window=32)
    if kind == "radius":
        vis = sparse_ref.radius_visible(frac, lat, n, cutoff)
    else:  # band in the sorted order, expressed on the original token order
        perm = plan.blocks.perm.cpu().long()
        band = sparse_ref.band_visible(N, n, 32)
        inv = torch.argsort(perm, dim=1)
        vis = torch.stack([band[b][inv[b]][:, inv[b]] for b in range(B)])
    bias = torch.zeros(B, N, N).masked_fill(~vis, torch.finfo(torch.float32).min)
    bias = bias[:, None].expand(-1, H, -1, -1).reshape(B * H, N, N).to(dev)
    res = []
    for sparse in (True, False):
        x = x0.to(dev).requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16, enabled=dtype == torch.bfloat16):
            if sparse:
                y = layer(x, key_padding_mask=pad.to(dev), sparse_plan=plan)
            else:
                y, _ = layer.attn(x, x, x, attn_mask=bias, need_weights=False)
        grads = torch.autograd.grad(y.float(), [x, *layer.parameters()], go.to(dev))
        res.append((y.float().cpu() * (~pad)[..., None], [t.float().cpu() for t in grads]))
    assert layer._last_core_used == kind
    (y1, g1), (y2, g2) = res
    assert (y1 - y2).abs().max() <= tol * max(1.0, y2.abs().max()), (y1 - y2).abs().max()
    for a, b2 in zip(g1, g2):
        assert (a - b2).abs().max() <= tol * max(1.0, b2.abs().max())


@pytest.mark.gpu
def test_periodic_trunk_runs_with_a_sparse_plan():
    """The trunk hands one plan to all of its MHA layers; simplicial layers are untouched.  Forward and backward
    run, padded rows stay zero, and a larger cutoff (every pair visible) reproduces the dense trunk."""
    from matterformer_b200.trunk import TransformerTrunk, plan_sparse_attention

    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    B, N, C, H = 2, 24, 128, 2
    trunk = TransformerTrunk(C, H, ["mha", "simplicial", "mha"], simplicial_impl="torch").to(dev)
    for blk in trunk.blocks:  # move the zero-initialised modulation off zero so that attention matters
        torch.nn.init.normal_(blk.ada_ln[-1].weight, std=0.05)
    x = torch.randn(B, N, C, device=dev, requires_grad=True)
    cond = torch.randn(B, C, device=dev)
    n = torch.tensor([24, 17], device=dev)
    pad = torch.arange(N, device=dev)[None, :] >= n[:, None]
    lat = torch.tensor([[2.0, 2.1, 2.2, 0.05, -0.1, 0.1]] * B, device=dev)
    frac = torch.rand(B, N, 3, device=dev)
    plan = plan_sparse_attention(frac, lat, pad, cutoff=3.0)
    y = trunk(x, cond, pad_mask=pad, sparse_plan=plan)
    y.sum().backward()
    assert torch.isfinite(y).all() and torch.isfinite(x.grad).all()
    assert y[pad].abs().max() == 0
    everything = plan_sparse_attention(frac, lat, pad, cutoff=100.0)
    dense = trunk(x, cond, pad_mask=pad)
    same = trunk(x, cond, pad_mask=pad, sparse_plan=everything)
    torch.testing.assert_close(same, dense, atol=1e-4, rtol=1e-4)
    assert (y - dense).abs().max() > 1e-3  # the 3 A cutoff really hides keys


@pytest.mark.gpu
def test_benchmark_trunk_bf16_step_matches_the_torch_attention_paths():
    """The benchmark's network (12 layers, d_model 512, 8 heads, MHA and 2-simplicial layers alternating) under bf16
    autocast on 64 molecules: one EDM loss and its gradients with this library's attention kernels against the
    same weights with ``simplicial_impl="torch"`` and the MHA layers on ``nn.MultiheadAttention``.  2e-2 of the
    largest value for the loss, the outputs and a sample of parameter gradients (bf16 round-off accumulates
    differently on the two paths over twelve layers)."""
    from matterformer_b200 import synthetic
    from matterformer_b200.dp import build_edm_net
    from matterformer_b200.trunk import EDMLoss, RegularAttention

    dev = torch.device("cuda:0")
    fast = build_edm_net(seed=0).to(dev)
    slow = build_edm_net(seed=0, simplicial_impl="torch").to(dev)
    slow.load_state_dict(fast.state_dict())
    for m in slow.modules():
        if isinstance(m, RegularAttention):
            m.impl = "torch"
    b = {k: v.to(dev) for k, v in synthetic.config5_batch(64, seed=3).items() if k != "num_atoms"}
    loss_fn = EDMLoss(sigma_data=1.0)
    results = []
    for net in (fast, slow):
        torch.manual_seed(77)  # the loss draws sigma and the noise from the global generator
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss, diag = loss_fn(net, b["atom_types"], b["coords"], b["pad_mask"])
        loss.backward()
        results.append((loss.detach().float(), {n: p.grad.float() for n, p in net.named_parameters() if p.grad is not None}))
    used = {type(m).__name__ + ":" + str(m._last_core_used) for m in fast.modules() if isinstance(m, RegularAttention)}
    assert used == {"RegularAttention:cuda"}
    (l1, g1), (l2, g2) = results
    assert abs(l1 - l2) <= 2e-2 * abs(l2), (float(l1), float(l2))
    names = sorted(g2)[:: max(1, len(g2) // 24)]  # two dozen tensors spread over the layers
    assert len(names) >= 12
    for n in names:
        err = (g1[n] - g2[n]).abs().max().item()
        assert err <= 2e-2 * max(g2[n].abs().max().item(), 1e-3 * max(v.abs().max().item() for v in g2.values())), n


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1, 8), (7, 40), (1000, 512), (29696, 2560), (1024, 3072), (33, 264), (0, 64)])
def test_column_sums_match_torch(rows, cols, dtype):
    """``mf_column_sums`` (the bias gradient of a Linear layer from its output gradient) against a float64 sum of the
    same values; the order of the additions is fixed, so a second run gives the same bits."""
    from matterformer_b200.fused import column_sums

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(rows * 31 + cols)
    x = (torch.randn(rows, cols, device=dev, generator=g) + 0.25).to(dtype)
    out = column_sums(x)
    assert out.dtype == torch.float32 and out.shape == (cols,)
    ref = x.double().sum(0)
    tol = 1e-5 * max(1.0, rows ** 0.5)
    torch.testing.assert_close(out.double(), ref, atol=tol * 4, rtol=1e-5)
    assert torch.equal(out, column_sums(x))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("rows,cols", [(1, 8), (37, 264), (2000, 2048)])
def test_gelu_kernels_match_torch(rows, cols, dtype, tol):
    """GELU (tanh form) forward, and backward with the column sums of the result, against ``F.gelu`` and autograd."""
    import torch.nn.functional as F
    from matterformer_b200.fused import gelu_tanh_backward, gelu_tanh_forward

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(rows + cols)
    pre = (torch.randn(rows, cols, device=dev, generator=g) * 2.0).to(dtype)
    dy = torch.randn(rows, cols, device=dev, generator=g).to(dtype)
    ref_in = pre.detach().clone().requires_grad_(True)
    ref = F.gelu(ref_in, approximate="tanh")
    (ref_dx,) = torch.autograd.grad(ref, ref_in, dy)
    y = gelu_tanh_forward(pre)
    dx, sums = gelu_tanh_backward(pre, dy)
    torch.testing.assert_close(y.float(), ref.float(), atol=tol, rtol=tol)
    torch.testing.assert_close(dx.float(), ref_dx.float(), atol=tol, rtol=tol)
    torch.testing.assert_close(sums.double(), dx.double().sum(0), atol=1e-4 * max(1.0, rows ** 0.5), rtol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("affine", [False, True])
def test_layer_norm_on_the_fused_kernels_matches_torch(affine):
    """``trunk.layer_norm`` evaluates an ``nn.LayerNorm`` (affine or not) with the LayerNorm-modulate kernels: output,
    input gradient and the gradients of weight and bias against the module itself."""
    from matterformer_b200.trunk import layer_norm

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(5)
    norm = torch.nn.LayerNorm(512, eps=1e-6, elementwise_affine=affine).to(dev)
    if affine:
        with torch.no_grad():
            norm.weight.add_(0.3 * torch.randn(512, device=dev, generator=g))
            norm.bias.add_(0.3 * torch.randn(512, device=dev, generator=g))
    x = torch.randn(6, 29, 512, device=dev, generator=g).requires_grad_(True)
    dy = torch.randn(6, 29, 512, device=dev, generator=g)
    params = list(norm.parameters())
    got = torch.autograd.grad(layer_norm(x, norm), [x] + params, dy)
    ref = torch.autograd.grad(norm(x), [x] + params, dy)
    torch.testing.assert_close(layer_norm(x, norm), norm(x), atol=1e-5, rtol=1e-5)
    for a, b in zip(got, ref):
        torch.testing.assert_close(a, b, atol=2e-4, rtol=1e-4)


@pytest.mark.gpu
def test_linear_gelu_bf16_matches_autocast():
    import torch.nn.functional as F
    from matterformer_b200.linear import linear_gelu_bf16

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(3)
    lin = torch.nn.Linear(64, 256).to(dev)
    x = torch.randn(6, 11, 64, device=dev, generator=g).bfloat16().requires_grad_(True)
    dy = torch.randn(6, 11, 256, device=dev, generator=g).bfloat16()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = linear_gelu_bf16(x, lin.weight, lin.bias)
        y_ref = F.gelu(F.linear(x, lin.weight, lin.bias), approximate="tanh")
    torch.testing.assert_close(y.float(), y_ref.float(), atol=1e-2, rtol=1e-2)
    got = torch.autograd.grad(y, [x, lin.weight, lin.bias], dy)
    ref = torch.autograd.grad(y_ref, [x, lin.weight, lin.bias], dy)
    assert got[1].dtype == torch.float32 and got[2].dtype == torch.float32
    for a, b in zip(got, ref):
        torch.testing.assert_close(a.float(), b.float(), atol=2e-2 * b.float().abs().max().item(), rtol=0)


@pytest.mark.gpu
def test_linear_bf16_matches_autocast_and_follows_parameter_updates():
    """``linear_bf16`` is ``F.linear`` under bf16 autocast without the per-call casts: same output, fp32 weight and
    bias gradients at least as close to the fp32 ones as autocast's, and a bf16 copy that follows in-place updates of
    the parameter, eagerly and inside a replayed CUDA graph."""
    import torch.nn.functional as F
    from matterformer_b200.linear import linear_bf16, refresh_bf16_copies

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    lin = torch.nn.Linear(96, 40).to(dev)
    x = torch.randn(5, 7, 96, device=dev, generator=g).bfloat16().requires_grad_(True)
    dy = torch.randn(5, 7, 40, device=dev, generator=g).bfloat16()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = linear_bf16(x, lin.weight, lin.bias)
        y_ref = F.linear(x, lin.weight, lin.bias)
    assert y.dtype == torch.bfloat16 and torch.equal(y, y_ref)
    gx, gw, gb = torch.autograd.grad(y, [x, lin.weight, lin.bias], dy)
    rx, rw, rb = torch.autograd.grad(y_ref, [x, lin.weight, lin.bias], dy)
    assert gw.dtype == torch.float32 and gb.dtype == torch.float32
    torch.testing.assert_close(gx.float(), rx.float(), atol=2e-2 * rx.float().abs().max().item(), rtol=0)
    w16, x32, dy32 = lin.weight.detach().bfloat16().float(), x.detach().float().reshape(-1, 96), dy.float().reshape(-1, 40)
    exact_w, exact_b = dy32.t() @ x32, dy32.sum(0)
    assert (gw - exact_w).abs().max() <= (rw - exact_w).abs().max() + 1e-6
    assert (gb - exact_b).abs().max() <= (rb - exact_b).abs().max() + 1e-6
    torch.testing.assert_close(gw, rw, atol=2e-2 * rw.abs().max().item(), rtol=0)
    # an optimizer-style in-place update is seen by the next call
    with torch.no_grad():
        lin.weight.mul_(0.5)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y2 = linear_bf16(x, lin.weight, lin.bias)
        y2_ref = F.linear(x, lin.weight, lin.bias)
    assert torch.equal(y2, y2_ref)
    # captured: the forced refresh is part of the graph, so replays follow updates made by other captured work
    params = [lin.weight, lin.bias]
    xs = x.detach()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        for _ in range(2):
            refresh_bf16_copies(params, force=True)
            out = linear_bf16(xs, lin.weight, lin.bias)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph), torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        refresh_bf16_copies(params, force=torch.cuda.is_current_stream_capturing())
        out = linear_bf16(xs, lin.weight, lin.bias)
        lin.weight.mul_(2.0)  # stands in for the optimizer step of a captured training step
    for _ in range(3):
        with torch.no_grad():
            expect = F.linear(xs, lin.weight.detach().bfloat16(), lin.bias.detach().bfloat16())
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, expect)


@pytest.mark.gpu
def test_trunk_bf16_step_runs_and_learns():
    dev = torch.device("cuda:0")
    net = build_edm_net(d_model=128, n_heads=2, n_layers=4, seed=0).to(dev)
    opt = torch.optim.AdamW(net.parameters(), lr=1e-3)
    batch = {k: v.to(dev) for k, v in config5_batch(64, seed=1).items() if k != "num_atoms"}
    loss_fn = EDMLoss(sigma_data=1.0)
    torch.manual_seed(0)
    g = torch.Generator(device=dev).manual_seed(0)
    sigma = torch.exp(torch.randn(64, device=dev, generator=g) * 1.2 - 1.2)
    losses = [float(edm_train_step(net, loss_fn, opt, batch, sigma=sigma)) for _ in range(8)]
    assert all(torch.isfinite(torch.tensor(losses))) and losses[-1] < losses[0]
    used = {m._last_impl_used for m in net.modules() if hasattr(m, "_last_impl_used")}
    assert used == {"cuda"}


def _dp_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        net = build_edm_net(d_model=32, n_heads=2, n_layers=2, simplicial_impl="torch", seed=0)
        with torch.no_grad():
            gen = torch.Generator().manual_seed(5)
            for p in net.parameters():
                p.add_(torch.randn(p.shape, generator=gen) * 0.05)
        ddp = wrap_data_parallel(net)
        full = {k: v for k, v in config5_batch(8, seed=3).items() if k != "num_atoms"}
        gen = torch.Generator().manual_seed(11)
        sigma = torch.exp(torch.randn(8, generator=gen) * 1.2 - 1.2)
        an = torch.randn(8, full["coords"].shape[1], 6, generator=gen)
        cn = torch.randn(8, full["coords"].shape[1], 3, generator=gen)
        mine = shard_batch({**full, "sigma": sigma, "an": an, "cn": cn}, rank, world)
        loss_fn = EDMLoss(sigma_data=1.0)
        loss, _ = loss_fn(ddp, mine["atom_types"], mine["coords"], mine["pad_mask"], sigma=mine["sigma"],
                          atom_noise=mine["an"], coord_noise=mine["cn"])  # fmt: skip
        loss.backward()
        if rank == 0:
            torch.save({k: p.grad.clone() for k, p in net.named_parameters()}, out)
    finally:
        dist.destroy_process_group()


def test_data_parallel_gradients_equal_full_batch(tmp_path):
    """Two gloo ranks on half the batch each: the all-reduced gradients equal the single-process full-batch ones."""
    out = str(tmp_path / "grads.pt")
    port = 29500 + os.getpid() % 2000
    mp.start_processes(_dp_worker, args=(2, port, out), nprocs=2, join=True, start_method="spawn")
    got = torch.load(out)
    net = build_edm_net(d_model=32, n_heads=2, n_layers=2, simplicial_impl="torch", seed=0)
    with torch.no_grad():
        gen = torch.Generator().manual_seed(5)
        for p in net.parameters():
            p.add_(torch.randn(p.shape, generator=gen) * 0.05)
    full = {k: v for k, v in config5_batch(8, seed=3).items() if k != "num_atoms"}
    gen = torch.Generator().manual_seed(11)
    sigma = torch.exp(torch.randn(8, generator=gen) * 1.2 - 1.2)
    an = torch.randn(8, full["coords"].shape[1], 6, generator=gen)
    cn = torch.randn(8, full["coords"].shape[1], 3, generator=gen)
    loss, _ = EDMLoss(sigma_data=1.0)(net, full["atom_types"], full["coords"], full["pad_mask"], sigma=sigma,
                                      atom_noise=an, coord_noise=cn)  # fmt: skip
    loss.backward()
    for k, p in net.named_parameters():
        torch.testing.assert_close(got[k], p.grad, atol=1e-5, rtol=1e-4, msg=lambda m, k=k: f"{k}: {m}")


def test_shard_batch_rejects_ragged_split():
    with pytest.raises(ValueError):
        shard_batch({"x": torch.zeros(5, 2)}, 0, 2)
