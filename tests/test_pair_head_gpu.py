"""Parity of the equivariant coordinate-head kernels (through the C ABI) with the CPU oracle and with the golden
vectors the reference model produced.  fp32 tolerance 1e-4 of the largest reference value per tensor; bf16 inputs
2e-2."""
import pytest
import torch
import torch.nn.functional as F

from matterformer_b200 import fused
from oracle.pair_head_ref import equivariant_coord_delta, rbf_constants

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
LEAVES = ("trunk_out", "w0", "b0", "w1", "b1")


def run_kernel(trunk_out, coords, pad, w0, b0, w1, b1, grad_out, *, dtype=torch.float32):
    """The composition the trunk uses: two per-atom GEMMs for the halves of the first Linear, then the kernel."""
    centers, gamma = rbf_constants()
    leaves = [t.to(DEV).requires_grad_(True) for t in (trunk_out, w0, b0, w1, b1)]
    h, w0d, b0d, w1d, b1d = leaves
    d = h.shape[-1]
    a = F.linear(h, w0d[:, :d]).to(dtype)
    b = F.linear(h, w0d[:, d : 2 * d], b0d).to(dtype)
    out = fused.equivariant_pair_head(a, b, coords.to(DEV), (~pad).to(DEV), w0d[:, 2 * d :], w1d, b1d,
                                      centers.to(DEV), float(gamma))  # fmt: skip
    grads = torch.autograd.grad(out, leaves, grad_out.to(DEV))
    torch.cuda.synchronize()
    return out.detach().cpu(), {n: g.cpu() for n, g in zip(LEAVES, grads)}


def run_oracle(trunk_out, coords, pad, w0, b0, w1, b1, grad_out):
    centers, gamma = rbf_constants()
    leaves = [t.clone().requires_grad_(True) for t in (trunk_out, w0, b0, w1, b1)]
    out = equivariant_coord_delta(leaves[0], coords, pad, *leaves[1:], centers, gamma)
    grads = torch.autograd.grad(out, leaves, grad_out)
    return out.detach(), dict(zip(LEAVES, grads))


def assert_close_scaled(a, b, tol, what):
    scale = max(float(b.abs().max()), 1e-3)
    err = float((a - b).abs().max())
    assert err <= tol * scale, f"{what}: max err {err:.3e} > {tol} * {scale:.3e}"


def random_case(B, N, d, seed, *, lo=1, holes=False):
    g = torch.Generator().manual_seed(seed)
    n = torch.randint(lo, N + 1, (B,), generator=g)
    n[0] = N
    pad = torch.arange(N)[None, :] >= n[:, None]
    if holes:
        pad |= torch.rand(B, N, generator=g) < 0.15
    coords = (torch.randn(B, N, 3, generator=g) * 1.5).masked_fill(pad[..., None], 0.0)
    trunk_out = torch.randn(B, N, d, generator=g)
    w0 = torch.randn(128, 2 * d + 16, generator=g) * (2 * d + 16) ** -0.5
    b0 = torch.randn(128, generator=g) * 0.1
    w1 = torch.randn(1, 128, generator=g) * 0.1
    b1 = torch.randn(1, generator=g) * 0.1
    grad_out = torch.randn(B, N, 3, generator=g)
    return trunk_out, coords, pad, w0, b0, w1, b1, grad_out


def test_matches_reference_golden(golden):
    g = golden("pair_head.npz")
    case = (g["trunk_out"], g["coords"], g["pad_mask"].bool(), g["w0"], g["b0"], g["w1"], g["b1"], g["grad_out"])
    out, grads = run_kernel(*case)
    assert_close_scaled(out, g["out"], 1e-4, "out")
    for n in LEAVES:
        assert_close_scaled(grads[n], g["d_" + n], 1e-4, "d" + n)
    pad = g["pad_mask"].bool()
    assert out[pad].abs().max() == 0  # exact zeros on padding, for a lone atom and for an empty molecule
    assert out[2].abs().max() == 0 and out[3].abs().max() == 0


@pytest.mark.parametrize("B,N,d,holes", [(3, 1, 16, False), (5, 8, 32, False), (7, 29, 64, True), (2, 64, 32, False),
                                         (2, 65, 32, True), (3, 150, 48, True), (300, 29, 16, False)])  # fmt: skip
def test_against_oracle(B, N, d, holes):
    case = random_case(B, N, d, seed=1000 + N + B, holes=holes)
    ref_out, ref_grads = run_oracle(*case)
    out, grads = run_kernel(*case)
    assert_close_scaled(out, ref_out, 1e-4, "out")
    for n in LEAVES:
        assert_close_scaled(grads[n], ref_grads[n], 2e-4, "d" + n)


def test_bf16_inputs():
    """bf16 a / b (what autocast hands over): fp32 arithmetic on the rounded vectors."""
    case = random_case(6, 29, 64, seed=5)
    ref_out, ref_grads = run_oracle(*case)
    out, grads = run_kernel(*case, dtype=torch.bfloat16)
    assert_close_scaled(out, ref_out, 2e-2, "out")
    for n in LEAVES:
        assert_close_scaled(grads[n], ref_grads[n], 2e-2, "d" + n)


def test_reproducible():
    case = random_case(40, 29, 32, seed=9, holes=True)
    first = run_kernel(*case)
    second = run_kernel(*case)
    assert torch.equal(first[0], second[0])
    for n in LEAVES:
        assert torch.equal(first[1][n], second[1][n])


def test_model_uses_the_kernel_and_agrees_with_its_torch_path():
    from matterformer_b200.trunk import EDMModel

    torch.manual_seed(0)
    model = EDMModel(d_model=64, n_heads=2, n_layers=1).to(DEV)
    with torch.no_grad():
        for p in model.pair_head.parameters():
            p.add_(torch.randn_like(p) * 0.1)
    B, N = 9, 23
    n = torch.randint(1, N + 1, (B,))
    pad = (torch.arange(N)[None, :] >= n[:, None]).to(DEV)
    coords = torch.randn(B, N, 3, device=DEV).masked_fill(pad[..., None], 0.0)
    h = torch.randn(B, N, 64, device=DEV, requires_grad=True)
    params = list(model.pair_head.parameters())
    go = torch.randn(B, N, 3, device=DEV)
    fast = model._coord_delta(h, coords, pad)
    slow = model._coord_delta_torch(h, coords, pad)
    assert fast.grad_fn is not None and "PairHead" in type(fast.grad_fn).__name__
    assert_close_scaled(fast.detach().cpu(), slow.detach().cpu(), 1e-4, "out")
    gf = torch.autograd.grad(fast, [h] + params, go)
    gs = torch.autograd.grad(slow, [h] + params, go)
    for i, (x, y) in enumerate(zip(gf, gs)):
        assert_close_scaled(x.cpu(), y.cpu(), 2e-4, f"grad {i}")
