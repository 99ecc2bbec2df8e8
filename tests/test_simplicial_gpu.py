"""Parity of the CUDA 2-simplicial attention kernels (through the C ABI) with the CPU oracle and with
the golden vectors the reference produced.  Tolerances: fp32 1e-4 (the reference's own GPU parity
bar, tests/test_simplicial_attention.py:886), bf16 2e-2 of the reference's largest value."""
import math

import pytest
import torch

import matterformer_b200 as mfb
from matterformer_b200 import simplicial as simplicial_mod
from matterformer_b200 import synthetic
from conftest import bf16_allowance
from oracle.simplicial_ref import SimplicialInputs, simplicial_forward, simplicial_forward_backward

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("q", "k1", "v1", "k2", "v2")


def run_cuda(inp: SimplicialInputs, grad_out, *, dtype=torch.float32, precision="ieee_fp32", backend="auto"):
    prev = mfb.set_backend(backend)
    try:
        t = [getattr(inp, n).to(DEV, dtype).requires_grad_(True) for n in NAMES]
        qv, kv = inp.query_valid.to(DEV), inp.pair_key_valid.to(DEV)
        pv = inp.pair_valid.to(DEV) if inp.pair_valid is not None else None
        out, lse, out32 = mfb.cuda_simplicial_attention_forward(
            *[x.detach() for x in t], query_valid=qv, pair_key_valid=kv, pair_valid=pv, precision=precision)  # fmt: skip
        y = mfb.simplicial_attention_cuda(*t, query_valid=qv, pair_key_valid=kv, pair_valid=pv, precision=precision)
        grads = torch.autograd.grad(y, t, grad_out.to(DEV, dtype))
        torch.cuda.synchronize()
        return out32.cpu(), lse.cpu(), {n: g.float().cpu() for n, g in zip(NAMES, grads)}, y.detach().float().cpu()
    finally:
        mfb.set_backend(prev)


def golden_inputs(g):
    valid = g["valid"].bool()
    return SimplicialInputs(q=g["in_q"], k1=g["in_k1"], v1=g["in_v1"], k2=g["in_k2"], v2=g["in_v2"], query_valid=valid,
                            pair_key_valid=valid, pair_valid=g["pair_valid"].bool() if "pair_valid" in g else None)  # fmt: skip


def assert_rel(a, b, tol, what):
    scale = max(1.0, b.abs().max().item()) if tol <= 1e-3 else b.abs().max().item()
    err = (a - b).abs().max().item()
    assert err <= tol * scale, f"{what}: max err {err:.3e} > {tol} * {scale:.3e}"


@pytest.mark.parametrize("name", ["pad", "holes", "peaked", "config1"])
def test_fp32_matches_reference_golden(golden, name):
    g = golden(f"simplicial_{name}.npz")
    inp = golden_inputs(g)
    out, lse, grads, y = run_cuda(inp, g["grad_out"])
    torch.testing.assert_close(out, g["out"], atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(y, g["out"], atol=1e-4, rtol=1e-4)
    for n in NAMES:
        torch.testing.assert_close(grads[n], g["d_" + n], atol=1e-4, rtol=1e-4, msg=lambda m, n=n: f"d{n}: {m}")
    _, lse_ref = simplicial_forward(inp, return_lse=True)
    torch.testing.assert_close(lse, lse_ref, atol=1e-4, rtol=1e-4)
    pad = ~inp.query_valid
    if pad.any():  # exact zeros on padded rows
        sel = pad[:, None, :].expand(-1, out.shape[1], -1)
        assert out[sel].abs().max() == 0
        for n in NAMES:
            assert grads[n][sel].abs().max() == 0


BIAS_NAMES = ("u", "v_bias", "w", "gate")


def run_cuda_bias(inp: SimplicialInputs, grad_out, *, dtype=torch.float32, precision="ieee_fp32"):
    """Forward and backward with the factorized bias; returns (out, {name: grad}) on the CPU in fp32."""
    t = [getattr(inp, n).to(DEV, dtype).requires_grad_(True) for n in NAMES]
    bias = [getattr(inp, n).to(DEV, dtype).requires_grad_(True) for n in BIAS_NAMES]
    qv, kv = inp.query_valid.to(DEV), inp.pair_key_valid.to(DEV)
    pv = inp.pair_valid.to(DEV) if inp.pair_valid is not None else None
    y = mfb.simplicial_attention_cuda(*t, query_valid=qv, pair_key_valid=kv, pair_valid=pv,
                                      factorized_bias=tuple(bias), precision=precision)  # fmt: skip
    grads = torch.autograd.grad(y, t + bias, grad_out.to(DEV, dtype))
    torch.cuda.synchronize()
    return y.detach().float().cpu(), {n: g.float().cpu() for n, g in zip(NAMES + BIAS_NAMES, grads)}


def test_factorized_bias_matches_reference_golden(golden):
    """logits += gate_i (u_ij + v_ik + w_jk): outputs and all nine gradients against the reference's."""
    g = golden("simplicial_factorized.npz")
    inp = golden_inputs(g)
    for n in BIAS_NAMES:
        setattr(inp, n, g["in_" + n])
    y, grads = run_cuda_bias(inp, g["grad_out"])
    torch.testing.assert_close(y, g["out"], atol=1e-4, rtol=1e-4)
    for n in NAMES + BIAS_NAMES:
        torch.testing.assert_close(grads[n], g["d_" + n], atol=1e-4, rtol=1e-4, msg=lambda m, n=n: f"d{n}: {m}")


@pytest.mark.parametrize("N,D,holes", [(5, 8, False), (33, 32, True), (70, 64, True)])
def test_factorized_bias_against_oracle(N, D, holes):
    inp, grad_out = _random_case(2, 3, N, D, seed=100 + N, scale=0.7, holes=holes, lo=max(1, N - 9))
    gen = torch.Generator().manual_seed(N)
    for n in ("u", "v_bias", "w"):
        setattr(inp, n, torch.randn(2, 3, N, N, generator=gen) * 0.5)
    inp.gate = torch.randn(2, 3, N, generator=gen)
    ref_out, ref_grads = simplicial_forward_backward(inp, grad_out)
    y, grads = run_cuda_bias(inp, grad_out)
    torch.testing.assert_close(y, ref_out, atol=1e-4, rtol=1e-4)
    for n in NAMES + BIAS_NAMES:
        torch.testing.assert_close(grads[n], ref_grads[n], atol=1e-4, rtol=1e-4, msg=lambda m, n=n: f"d{n}: {m}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_factorized_bias_cancellation(dtype):
    """u ~ +1000 and v ~ -1000 with gate 1: the three bias terms must be summed in fp32 before they meet the logits
    (the stress input of scripts/diagnose_simplicial_triton_parity.py:80-84; fp32 summation is pinned by
    tests/test_simplicial_attention.py:299-311).  A kernel that adds them one at a time to a bf16 or scaled logit, or
    applies the gate per term, loses the 0.2-sized signal under the 1000-sized offsets."""
    B, H, N, D = 2, 2, 24, 16
    inp, grad_out = _random_case(B, H, N, D, seed=77, scale=0.7, holes=False, lo=N - 5)
    gen = torch.Generator().manual_seed(78)
    inp.u = 1000.0 + 0.2 * torch.randn(B, H, N, N, generator=gen)
    inp.v_bias = -1000.0 + 0.2 * torch.randn(B, H, N, N, generator=gen)
    inp.w = 0.2 * torch.randn(B, H, N, N, generator=gen)
    inp.gate = torch.ones(B, H, N)
    if dtype == torch.bfloat16:  # the operands the kernel sees are the rounded ones; the oracle gets the same values
        for n in NAMES + BIAS_NAMES:
            setattr(inp, n, getattr(inp, n).to(dtype).float())
    if dtype == torch.bfloat16:
        grad_out = grad_out.bfloat16().float()
    ref_out, ref_grads = simplicial_forward_backward(inp, grad_out)
    y, grads = run_cuda_bias(inp, grad_out, dtype=dtype, precision="ieee_fp32" if dtype == torch.float32 else "bf16_tc")
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(y, ref_out, atol=tol, rtol=tol)
    for n in NAMES + BIAS_NAMES:
        scale = max(float(ref_grads[n].abs().max()), 1.0)
        torch.testing.assert_close(grads[n], ref_grads[n], atol=tol * scale, rtol=tol, msg=lambda m, n=n: f"d{n}: {m}")


RES_NAMES = ("angle_left", "angle_right", "angle_gate", "message_left", "message_right", "message_basis")


def run_cuda_all_bias(inp: SimplicialInputs, grad_out, *, with_factorized=True):
    """Forward and backward with every geometry operand the reference interface has."""
    t = [getattr(inp, n).to(DEV).requires_grad_(True) for n in NAMES]
    qv, kv = inp.query_valid.to(DEV), inp.pair_key_valid.to(DEV)
    pv = inp.pair_valid.to(DEV) if inp.pair_valid is not None else None
    extra_names = (BIAS_NAMES if with_factorized else ()) + RES_NAMES
    extra = {n: getattr(inp, n).to(DEV).requires_grad_(True) for n in extra_names}
    y = mfb.simplicial_attention_cuda(
        *t, query_valid=qv, pair_key_valid=kv, pair_valid=pv, precision="ieee_fp32",
        factorized_bias=tuple(extra[n] for n in BIAS_NAMES) if with_factorized else None,
        angle_residual=(extra["angle_left"], extra["angle_right"], extra["angle_gate"]),
        message_residual=(extra["message_left"], extra["message_right"], extra["message_basis"]))  # fmt: skip
    grads = torch.autograd.grad(y, t + list(extra.values()), grad_out.to(DEV))
    torch.cuda.synchronize()
    return y.detach().cpu(), {n: g.cpu() for n, g in zip(NAMES + extra_names, grads)}


def test_all_geometry_operands_match_reference_golden(golden):
    """Factorized bias + low-rank angle + low-rank message together: output and all 15 gradients."""
    g = golden("simplicial_bias.npz")
    inp = golden_inputs(g)
    for n in BIAS_NAMES + RES_NAMES:
        setattr(inp, n, g["in_" + n])
    y, grads = run_cuda_all_bias(inp, g["grad_out"])
    torch.testing.assert_close(y, g["out"], atol=1e-4, rtol=1e-4)
    for n in NAMES + BIAS_NAMES + RES_NAMES:
        torch.testing.assert_close(grads[n], g["d_" + n], atol=1e-4, rtol=1e-4, msg=lambda m, n=n: f"d{n}: {m}")


@pytest.mark.parametrize("N,D,ra,rm,holes", [(6, 8, 1, 1, False), (37, 32, 16, 16, True), (70, 64, 32, 7, True)])
def test_low_rank_residuals_against_oracle(N, D, ra, rm, holes):
    B, H = 2, 3
    inp, grad_out = _random_case(B, H, N, D, seed=300 + N, scale=0.7, holes=holes, lo=max(1, N - 9))
    gen = torch.Generator().manual_seed(N + 1)
    inp.angle_left = torch.randn(B, H, N, N, ra, generator=gen)
    inp.angle_right = torch.randn(B, H, N, N, ra, generator=gen)
    inp.angle_gate = torch.randn(B, H, N, generator=gen)
    inp.message_left = torch.randn(B, H, N, N, rm, generator=gen)
    inp.message_right = torch.randn(B, H, N, N, rm, generator=gen)
    inp.message_basis = torch.randn(H, rm, D, generator=gen) / D**0.5
    ref_out, ref_grads = simplicial_forward_backward(inp, grad_out)
    y, grads = run_cuda_all_bias(inp, grad_out, with_factorized=False)
    torch.testing.assert_close(y, ref_out, atol=1e-4, rtol=1e-4)
    for n in NAMES + RES_NAMES:
        scale = max(1.0, ref_grads[n].abs().max().item())
        err = (grads[n] - ref_grads[n]).abs().max().item()
        assert err <= 1e-4 * scale, f"d{n}: max err {err:.3e} > 1e-4 * {scale:.3e}"


def test_factorized_bias_bf16_other_head_dims_run_on_cuda_cores():
    """bf16 inputs with a bias and a head_dim other than 64 take the CUDA-core kernel (fp32 arithmetic on rounded
    inputs)."""
    inp, grad_out = _random_case(2, 2, 48, 32, seed=7, scale=0.5, lo=40)
    gen = torch.Generator().manual_seed(5)
    for n in ("u", "v_bias", "w"):
        setattr(inp, n, (torch.randn(2, 2, 48, 48, generator=gen) * 0.5).bfloat16().float())
    inp.gate = torch.randn(2, 2, 48, generator=gen).bfloat16().float()
    for n in NAMES:
        setattr(inp, n, getattr(inp, n).bfloat16().float())
    ref_out, ref_grads = simplicial_forward_backward(inp, grad_out.bfloat16().float())
    y, grads = run_cuda_bias(inp, grad_out, dtype=torch.bfloat16, precision="bf16_tc")
    assert_rel(y, ref_out, 2e-2, "out")
    for n in NAMES + BIAS_NAMES:
        assert_rel(grads[n], ref_grads[n], 2e-2, f"d{n}")


def test_known_answer(golden):
    g = golden("simplicial_known_answer.npz")
    ones = torch.ones(1, 2, dtype=torch.bool)
    inp = SimplicialInputs(q=g["q"], k1=g["k1"], v1=g["v1"], k2=g["k2"], v2=g["v2"], query_valid=ones,
                           pair_key_valid=ones, pair_valid=g["pair_valid"].bool())  # fmt: skip
    out, lse, _, _ = run_cuda(inp, torch.ones(1, 1, 2, 2))
    torch.testing.assert_close(out[0, 0], torch.tensor([[3.0, 10.0], [3.0, 10.0]]))
    assert lse.abs().max() == 0


def _random_case(B, H, N, D, seed, scale=1.0, holes=False, lo=None):
    g = torch.Generator().manual_seed(seed)
    t = {n: torch.randn(B, H, N, D, generator=g) * scale for n in NAMES}
    go = torch.randn(B, H, N, D, generator=g)
    n_valid = torch.randint(lo if lo is not None else max(1, N // 2), N + 1, (B,), generator=g)
    valid = torch.arange(N)[None, :] < n_valid[:, None]
    pv = (torch.rand(B, N, N, generator=g) > 0.4) if holes else None
    return SimplicialInputs(**t, query_valid=valid, pair_key_valid=valid, pair_valid=pv), go


@pytest.mark.parametrize("N", [1, 2, 3, 5, 7, 31, 32, 33, 63, 65])
@pytest.mark.parametrize("D", [8, 16, 32, 64, 128])
def test_fp32_small_exhaustive(N, D):
    if N > 33 and D not in (32, 64):
        pytest.skip("large N only at the common head sizes")
    inp, go = _random_case(2, 2, N, D, seed=100 * N + D, scale=D**-0.25, holes=(N % 2 == 1))
    out_ref, g_ref = simplicial_forward_backward(inp, go)
    out, _, grads, _ = run_cuda(inp, go)
    assert_rel(out, out_ref, 1e-4, "out")
    for n in NAMES:
        assert_rel(grads[n], g_ref[n], 1e-4, "d" + n)


def test_masked_members_cannot_influence(golden):
    """Huge values on excluded keys leave the result untouched (reference tests/...:415-445)."""
    inp, go = _random_case(1, 2, 9, 16, seed=7, holes=True)
    inp.pair_key_valid = inp.pair_key_valid.clone()
    inp.pair_key_valid[0, 2] = False
    base, _, gbase, _ = run_cuda(inp, go)
    for n in ("k1", "v1", "k2", "v2"):
        t = getattr(inp, n).clone()
        t[:, :, 2] = 1000.0
        setattr(inp, n, t)
    out, _, grads, _ = run_cuda(inp, go)
    assert torch.equal(out, base)
    assert torch.equal(grads["q"], gbase["q"])


def test_fully_masked_and_empty():
    inp, go = _random_case(2, 1, 6, 8, seed=9)
    inp.pair_key_valid = torch.zeros_like(inp.pair_key_valid)  # no visible pair anywhere
    out, lse, grads, _ = run_cuda(inp, go)
    assert out.abs().max() == 0 and lse.abs().max() == 0
    for n in NAMES:
        assert grads[n].abs().max() == 0
    # zero-sized batch
    z = torch.zeros(0, 2, 4, 8, device=DEV)
    ok = torch.ones(0, 4, dtype=torch.bool, device=DEV)
    o, l, _ = mfb.cuda_simplicial_attention_forward(z, z, z, z, z, query_valid=ok, pair_key_valid=ok, pair_valid=None)
    assert o.shape == (0, 2, 4, 8) and l.shape == (0, 2, 4)


def test_tensor_maps_are_in_use():
    """On a GPU box the driver's tensor-map encoder is found, so K2 / V2 tiles travel by bulk tensor copies."""
    from matterformer_b200 import _lib

    assert _lib.lib().mf_feature_flags() & 1


def test_host_pipeline_gives_the_direct_results():
    """Copies and kernels on three streams, several steps in flight: every step's host outputs equal the
    results of the plain calls on the same inputs, bit for bit (the kernels are deterministic)."""
    t = synthetic.config2(seed=3, batch=4)
    names = NAMES + ("grad_out",)
    valid = t["valid"].to(DEV)
    pipe = mfb.HostPipelinedSimplicial(torch.device(DEV), query_valid=valid, pair_key_valid=valid)
    steps = []
    for s_i in range(5):  # different inputs per step, so that a mixed-up buffer would show
        host_in = [(t[n].float() * (1.0 + 0.1 * s_i)).to(t[n].dtype).pin_memory() for n in names]
        host_out = [torch.empty_like(t["q"]).pin_memory() for _ in range(6)]
        pipe.submit(host_in, host_out)
        steps.append((host_in, host_out))
    pipe.finish()
    for host_in, host_out in steps:
        d = [h.to(DEV) for h in host_in]
        out, lse, out32 = mfb.cuda_simplicial_attention_forward(*d[:5], query_valid=valid, pair_key_valid=valid,
                                                                pair_valid=None)  # fmt: skip
        grads = mfb.cuda_simplicial_attention_backward(d[5], *d[:5], out32, lse, query_valid=valid,
                                                       pair_key_valid=valid, pair_valid=None)  # fmt: skip
        for got, want in zip(host_out, (out, *grads[:5])):
            assert torch.equal(got, want.cpu())


def test_status_word_is_read_from_tensor_core_calls_only():
    """The CUDA-core kernels keep no status word: their scratch must not be mistaken for one."""
    inp, go = _random_case(2, 4, 40, 64, seed=3, scale=1 / 8.0, lo=30)
    for n in NAMES:
        setattr(inp, n, getattr(inp, n).bfloat16().float())
    run_cuda(inp, go, dtype=torch.bfloat16, precision="bf16_tc", backend="auto")
    assert simplicial_mod.device_status() == 0
    run_cuda(inp, go, dtype=torch.bfloat16, precision="bf16_tc", backend="generic")
    assert simplicial_mod.device_status() == 0


def test_deterministic():
    inp, go = _random_case(2, 2, 40, 32, seed=3)
    a = run_cuda(inp, go)
    b = run_cuda(inp, go)
    assert torch.equal(a[0], b[0])
    for n in NAMES:
        assert torch.equal(a[2][n], b[2][n])


@pytest.mark.parametrize("backend", ["generic", "auto"])
@pytest.mark.parametrize("N,lo", [(40, 20), (128, 100), (192, 130), (181, 150)])
def test_bf16_against_fp32_core_oracle(backend, N, lo):
    inp, go = _random_case(2, 2, N, 64, seed=N, scale=1 / 8.0, lo=lo)
    for n in NAMES:
        setattr(inp, n, getattr(inp, n).bfloat16().float())  # both sides see bf16-rounded inputs
    go = go.bfloat16().float()
    out_ref, g_ref = simplicial_forward_backward(inp, go)
    out, _, grads, y = run_cuda(inp, go, dtype=torch.bfloat16, precision="bf16_tc", backend=backend)
    assert_rel(out, out_ref, 2e-2, "out")
    assert_rel(y, out_ref, 2e-2, "out(bf16)")
    for n in NAMES:
        assert_rel(grads[n], g_ref[n], 2e-2, "d" + n)


@pytest.mark.parametrize("H", [4, 8])
@pytest.mark.parametrize("N,lo,holes,scale", [(5, 1, False, 1.0), (29, 9, False, 1 / 8.0), (29, 9, True, 1.0),
                                              (32, 30, True, 0.5), (17, 1, True, 0.5)])
def test_bf16_small_molecules_share_a_tile(H, N, lo, holes, scale):
    """At most 32 tokens: four heads of a molecule are packed into one 128-row tile of the tensor-core kernels.
    Heads must not leak into each other: every head gets different inputs, and results are checked per element."""
    inp, go = _random_case(5, H, N, 64, seed=1000 + N + H, scale=scale, holes=holes, lo=lo)
    for n in NAMES:
        setattr(inp, n, getattr(inp, n).bfloat16().float())
    go = go.bfloat16().float()
    out_ref, g_ref = simplicial_forward_backward(inp, go)
    _, lse_ref = simplicial_forward(inp, return_lse=True)
    out, lse, grads, y = run_cuda(inp, go, dtype=torch.bfloat16, precision="bf16_tc", backend="auto")
    assert_rel(out, out_ref, 2e-2, "out")
    assert_rel(y, out_ref, 2e-2, "out(bf16)")
    torch.testing.assert_close(lse, lse_ref, atol=3e-2, rtol=1e-2)
    allow = bf16_allowance(inp, go, out_ref, g_ref)  # 2e-2, or the reference's own bf16 path error if larger
    for n in NAMES:
        assert_rel(grads[n], g_ref[n], allow[n], "d" + n)
    pad = ~inp.query_valid
    if pad.any():  # exact zeros on padded rows
        sel = pad[:, None, :].expand(-1, H, -1)
        assert out[sel].abs().max() == 0
        for n in NAMES:
            assert grads[n][sel].abs().max() == 0
    assert simplicial_mod.device_status() == 0


@pytest.mark.parametrize("H", [4, 8])
@pytest.mark.parametrize("N,lo,holes", [(5, 1, False), (29, 9, False), (29, 9, True), (32, 30, True), (17, 1, True)])
def test_bf16_factorized_bias_inside_the_tile_kernels(H, N, lo, holes):
    """At most 32 tokens and a multiple of four heads: the factorized bias is added inside the tensor-core tile kernels
    (logits += gate_i ((u_ij + v_ik) + w_jk), summed in fp32) and its four gradients come out of the same backward
    kernel.  Outputs and all nine gradients against the oracle on the rounded inputs."""
    B = 5
    inp, go = _random_case(B, H, N, 64, seed=2000 + N + H, scale=0.5, holes=holes, lo=lo)
    gen = torch.Generator().manual_seed(N * 10 + H)
    for n in ("u", "v_bias", "w"):
        setattr(inp, n, (torch.randn(B, H, N, N, generator=gen) * 0.5).bfloat16().float())
    inp.gate = torch.randn(B, H, N, generator=gen).bfloat16().float()
    for n in NAMES:
        setattr(inp, n, getattr(inp, n).bfloat16().float())
    go = go.bfloat16().float()
    ref_out, ref_grads = simplicial_forward_backward(inp, go)
    y, grads = run_cuda_bias(inp, go, dtype=torch.bfloat16, precision="bf16_tc")
    assert simplicial_mod.device_status() == 0
    assert_rel(y, ref_out, 2e-2, "out")
    for n in NAMES + BIAS_NAMES:
        assert_rel(grads[n], ref_grads[n], 2.5e-2, f"d{n}")
    y2, grads2 = run_cuda_bias(inp, go, dtype=torch.bfloat16, precision="bf16_tc")
    assert torch.equal(y, y2) and all(torch.equal(grads[n], grads2[n]) for n in NAMES + BIAS_NAMES)
    pad = ~inp.query_valid
    if pad.any():  # padded rows: zero outputs and zero gradients, the bias gradients included
        sel = pad[:, None, :].expand(-1, H, -1)
        assert y[sel].abs().max() == 0
        for n in ("q", "u", "v_bias", "gate"):
            assert grads[n][sel].abs().max() == 0


@pytest.mark.parametrize("B,H,N,lo,holes", [(3, 3, 29, 9, False), (2, 2, 48, 40, True), (2, 2, 70, 50, True),
                                            (2, 1, 150, 120, True), (2, 2, 192, 150, False), (2, 2, 181, 130, True)])
def test_bf16_factorized_bias_one_head_per_tile(B, H, N, lo, holes):
    """More than 32 tokens, or heads that are not a multiple of four: the bias goes through the tile kernels with one
    head per tile.  Covers one and two query tiles / key slabs, token counts that are and are not multiples of four
    (vector and scalar additions into dv_bias), pair masks with holes; outputs and all nine gradients against the
    oracle on the rounded inputs, and bit-identical results on a second run."""
    inp, go = _random_case(B, H, N, 64, seed=3000 + N + H, scale=0.4, holes=holes, lo=lo)
    gen = torch.Generator().manual_seed(N * 10 + H)
    for n in ("u", "v_bias", "w"):
        setattr(inp, n, (torch.randn(B, H, N, N, generator=gen) * 0.5).bfloat16().float())
    inp.gate = torch.randn(B, H, N, generator=gen).bfloat16().float()
    for n in NAMES:
        setattr(inp, n, getattr(inp, n).bfloat16().float())
    go = go.bfloat16().float()
    ref_out, ref_grads = simplicial_forward_backward(inp, go)
    y, grads = run_cuda_bias(inp, go, dtype=torch.bfloat16, precision="bf16_tc")
    assert simplicial_mod.device_status() == 0
    assert_rel(y, ref_out, 2e-2, "out")
    for n in NAMES + BIAS_NAMES:
        assert_rel(grads[n], ref_grads[n], 2.5e-2, f"d{n}")
    y2, grads2 = run_cuda_bias(inp, go, dtype=torch.bfloat16, precision="bf16_tc")
    assert torch.equal(y, y2)
    for n in NAMES + BIAS_NAMES:
        assert torch.equal(grads[n], grads2[n]), n


@pytest.mark.parametrize("N,H", [(29, 4), (70, 2)])
def test_bf16_factorized_bias_gradients_are_optional(N, H):
    """The reference asks only for the bias gradients autograd needs (need_du ... need_dgate follow needs_input_grad,
    simplicial_attention.py:560-575): with u and gate alone requiring a gradient the tile kernels get NULL for the
    other two and must return the same du and dgate."""
    B = 2
    inp, go = _random_case(B, H, N, 64, seed=4000 + N, scale=0.4, holes=True, lo=N - 9)
    gen = torch.Generator().manual_seed(N)
    t = [getattr(inp, n).to(DEV, torch.bfloat16).requires_grad_(True) for n in NAMES]
    u, v, w = [(torch.randn(B, H, N, N, generator=gen) * 0.5).to(DEV) for _ in range(3)]
    gate = torch.randn(B, H, N, generator=gen).to(DEV)
    qv, kv, pv = inp.query_valid.to(DEV), inp.pair_key_valid.to(DEV), inp.pair_valid.to(DEV)

    def run(needs):
        bias = [x.clone().requires_grad_(r) for x, r in zip((u, v, w, gate), needs)]
        y = mfb.simplicial_attention_cuda(*t, query_valid=qv, pair_key_valid=kv, pair_valid=pv,
                                          factorized_bias=tuple(bias), precision="bf16_tc")  # fmt: skip
        wanted = [b for b in bias if b.requires_grad]
        return y, torch.autograd.grad(y, t + wanted, go.to(DEV, torch.bfloat16))

    y_all, g_all = run((True, True, True, True))
    y_two, g_two = run((True, False, False, True))
    assert simplicial_mod.device_status() == 0
    assert torch.equal(y_all, y_two)
    for a, b in zip(g_all[:5], g_two[:5]):
        assert torch.equal(a, b)
    assert torch.equal(g_all[5], g_two[5]) and torch.equal(g_all[8], g_two[6])  # du, dgate


def test_bf16_factorized_bias_tile_kernels_match_reference_golden(golden):
    """Outputs and all nine gradients of the reference (fp32, on bf16-exact operands: 3 molecules of 29 / 20 / 11 atoms,
    4 heads, head_dim 64, pair mask with holes) against the tensor-core tile kernels, within 2e-2 of each tensor's
    largest value."""
    g = golden("simplicial_factorized_tiles.npz")
    inp = golden_inputs(g)
    for n in BIAS_NAMES:
        setattr(inp, n, g["in_" + n])
    y, grads = run_cuda_bias(inp, g["grad_out"], dtype=torch.bfloat16, precision="bf16_tc")
    assert simplicial_mod.device_status() == 0
    assert_rel(y, g["out"], 2e-2, "out")
    for n in NAMES + BIAS_NAMES:
        assert_rel(grads[n], g["d_" + n], 2e-2, f"d{n}")


def test_bf16_factorized_bias_cancellation_inside_the_tile_kernels():
    """The +1000 / -1000 stress input at a shape the tile kernels take (four heads, 24 tokens, head_dim 64)."""
    B, H, N, D = 2, 4, 24, 64
    inp, go = _random_case(B, H, N, D, seed=79, scale=0.5, holes=False, lo=N - 5)
    gen = torch.Generator().manual_seed(80)
    inp.u = 1000.0 + 0.2 * torch.randn(B, H, N, N, generator=gen)
    inp.v_bias = -1000.0 + 0.2 * torch.randn(B, H, N, N, generator=gen)
    inp.w = 0.2 * torch.randn(B, H, N, N, generator=gen)
    inp.gate = torch.ones(B, H, N)
    for n in NAMES + BIAS_NAMES:
        setattr(inp, n, getattr(inp, n).bfloat16().float())
    go = go.bfloat16().float()
    ref_out, ref_grads = simplicial_forward_backward(inp, go)
    y, grads = run_cuda_bias(inp, go, dtype=torch.bfloat16, precision="bf16_tc")
    assert simplicial_mod.device_status() == 0
    torch.testing.assert_close(y, ref_out, atol=2e-2, rtol=2e-2)
    for n in NAMES + BIAS_NAMES:
        scale = max(float(ref_grads[n].abs().max()), 1.0)
        torch.testing.assert_close(grads[n], ref_grads[n], atol=2e-2 * scale, rtol=2e-2, msg=lambda m, n=n: f"d{n}: {m}")


def test_bf16_packed_heads_with_an_empty_molecule():
    """Four heads per tile, one molecule of the batch without a single valid token and one with a single token: the
    kernels that write their gradients themselves must leave exact zeros for the empty one."""
    B, H, N = 4, 4, 19
    inp, go = _random_case(B, H, N, 64, seed=4242, scale=0.5, holes=False, lo=5)
    inp.query_valid[1] = False
    inp.pair_key_valid[1] = False
    inp.query_valid[2] = False
    inp.pair_key_valid[2] = False
    inp.query_valid[2, 0] = True
    inp.pair_key_valid[2, 0] = True
    for n in NAMES:
        setattr(inp, n, getattr(inp, n).bfloat16().float())
    go = go.bfloat16().float()
    out_ref, g_ref = simplicial_forward_backward(inp, go)
    out, lse, grads, y = run_cuda(inp, go, dtype=torch.bfloat16, precision="bf16_tc", backend="auto")
    assert simplicial_mod.device_status() == 0
    assert_rel(out, out_ref, 2e-2, "out")
    allow = bf16_allowance(inp, go, out_ref, g_ref)
    for n in NAMES:
        assert_rel(grads[n], g_ref[n], allow[n], "d" + n)
        assert grads[n][1].abs().max() == 0, n
        assert grads[n][2, :, 1:].abs().max() == 0, n


@pytest.mark.parametrize("backend", ["generic", "auto"])
def test_bf16_peaked_softmax(backend):
    """Scaled-up queries make the softmax sharp, which exercises the running-maximum logic."""
    inp, go = _random_case(1, 2, 150, 64, seed=5, scale=1 / 8.0, holes=True, lo=140)
    inp.q = inp.q * 48.0
    for n in NAMES:
        setattr(inp, n, getattr(inp, n).bfloat16().float())
    go = go.bfloat16().float()
    out_ref, g_ref = simplicial_forward_backward(inp, go)
    out, _, grads, _ = run_cuda(inp, go, dtype=torch.bfloat16, precision="bf16_tc", backend=backend)
    allow = bf16_allowance(inp, go, out_ref, g_ref)  # 2e-2, or the reference's own bf16 path error if larger
    assert_rel(out, out_ref, allow["out"], "out")
    for n in NAMES:
        assert_rel(grads[n], g_ref[n], allow[n], "d" + n)


def test_config2_properties():
    """Full benchmark size (B=64, N=192, H=8, D=64, bf16): size-independent checks plus an oracle
    comparison on two molecules."""
    t = synthetic.config2(seed=0)
    dev = {n: t[n].to(DEV) for n in NAMES}
    valid = t["valid"].to(DEV)
    out, lse, out32 = mfb.cuda_simplicial_attention_forward(*[dev[n] for n in NAMES], query_valid=valid,
                                                            pair_key_valid=valid, pair_valid=None)  # fmt: skip
    assert torch.isfinite(out32).all() and torch.isfinite(lse).all()
    assert out32[~valid[:, None, :].expand(-1, 8, -1)].abs().max() == 0
    # linearity in v1: out(2*v1) = 2*out(v1) exactly (power-of-two scaling commutes with every rounding)
    out2, _, out2_32 = mfb.cuda_simplicial_attention_forward(dev["q"], dev["k1"], dev["v1"] * 2, dev["k2"], dev["v2"],
                                                             query_valid=valid, pair_key_valid=valid, pair_valid=None)  # fmt: skip
    assert torch.equal(out2_32, out32 * 2)
    # batch independence: molecules 3 and 17 alone give the same bits
    sel = torch.tensor([3, 17], device=DEV)
    o_s, _, o_s32 = mfb.cuda_simplicial_attention_forward(*[dev[n][sel] for n in NAMES], query_valid=valid[sel],
                                                          pair_key_valid=valid[sel], pair_valid=None)  # fmt: skip
    assert torch.equal(o_s32, out32[sel])
    inp = SimplicialInputs(**{n: t[n][[3, 17]].float() for n in NAMES}, query_valid=t["valid"][[3, 17]],
                           pair_key_valid=t["valid"][[3, 17]])  # fmt: skip
    ref = simplicial_forward(inp)
    assert_rel(o_s32.cpu(), ref, 2e-2, "config2 out")


def test_bounded_wait_gives_up_and_reports():
    """A wait on a barrier that is never signalled, with a limit of 50 000 clocks instead of the production second:
    the kernel sets the timeout status and returns (the path every tensor-core kernel takes when a hand-off never
    arrives); the context stays usable."""
    import ctypes

    from matterformer_b200 import _lib

    status = torch.full((2,), -7, dtype=torch.int32, device=DEV)
    _lib.check(_lib.lib().mf_selftest_wait_timeout(status.data_ptr(), 50_000, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    code, waited = status.tolist()
    assert code == _lib.MF_ERR_DEVICE_TIMEOUT
    assert 50_000 <= waited < 50_000_000
    assert torch.ones(4, device=DEV).sum().item() == 4.0  # the device still answers


def test_checked_mode_and_unaligned_views():
    """``set_check_status(True)`` reads the status word after every tensor-core call; a view that starts two bytes
    into a buffer is served by the element-wise kernel with the same results."""
    inp, go = _random_case(2, 2, 40, 64, seed=3, scale=1 / 8.0, lo=30)
    x = [getattr(inp, n).bfloat16().to(DEV) for n in NAMES]
    qv = inp.query_valid.to(DEV)
    prev = simplicial_mod.set_check_status(True)
    try:
        out, lse, out32 = mfb.cuda_simplicial_attention_forward(*x, query_valid=qv, pair_key_valid=qv, pair_valid=None)
    finally:
        simplicial_mod.set_check_status(prev)
    assert simplicial_mod.device_status() == 0
    buf = torch.empty(x[0].numel() + 1, dtype=torch.bfloat16, device=DEV)
    shifted = buf[1:].view_as(x[0])
    shifted.copy_(x[0])
    assert shifted.data_ptr() % 16 == 2 and shifted.is_contiguous()
    out_s, _, out32_s = mfb.cuda_simplicial_attention_forward(shifted, *x[1:], query_valid=qv, pair_key_valid=qv, pair_valid=None)
    assert_rel(out32_s.cpu(), out32.cpu(), 2e-2, "unaligned q")


@pytest.mark.parametrize("B,H,N,holes", [(3, 4, 29, False), (2, 8, 32, True), (5, 4, 7, False), (2, 4, 1, False)])
def test_packed_projection_matches_the_head_major_call(B, H, N, holes):
    """The entry points that read q, k1, v1, k2, v2 inside the (B,N,5,H,D) projection and write (B,N,H*D) and one
    packed gradient: bit for bit the head-major call on the split tensors (same kernels, other addresses), forward
    and all five gradients, and against the oracle within the bf16 allowance."""
    D = 64
    g = torch.Generator().manual_seed(31 * B + N)
    proj = (torch.randn(B, N, 5 * H * D, generator=g) * 0.7).bfloat16()
    grad_out = torch.randn(B, N, H * D, generator=g).bfloat16()
    n = torch.randint(1, N + 1, (B,), generator=g)
    n[0] = N
    valid = torch.arange(N)[None, :] < n[:, None]
    if holes:
        valid &= torch.rand(B, N, generator=g) > 0.2
        valid[:, 0] = True
    pair_valid = (valid[:, :, None] & valid[:, None, :]) if holes else None
    pd = proj.to(DEV).requires_grad_(True)
    qv = valid.to(DEV)
    pvd = pair_valid.to(DEV) if pair_valid is not None else None
    out = simplicial_mod.simplicial_attention_packed(pd, heads=H, query_valid=qv, pair_key_valid=qv, pair_valid=pvd)
    (gp,) = torch.autograd.grad(out, [pd], grad_out.to(DEV))
    assert mfb.simplicial.device_status() == 0
    # the same computation on split, scaled, head-major tensors
    parts = [proj.view(B, N, 5, H, D)[:, :, i].transpose(1, 2).contiguous() for i in range(5)]
    parts[0] = (parts[0].float() * 0.125).bfloat16()  # exact: a power of two
    t = [x.to(DEV).requires_grad_(True) for x in parts]
    prev = mfb.set_backend("tcgen05_tiles")
    try:
        y = mfb.simplicial_attention_cuda(*t, query_valid=qv, pair_key_valid=qv, pair_valid=pvd)
        grads = torch.autograd.grad(y, t, grad_out.view(B, N, H, D).transpose(1, 2).contiguous().to(DEV))
    finally:
        mfb.set_backend(prev)
    assert torch.equal(out.view(B, N, H, D).transpose(1, 2), y)
    want = torch.stack([gr.transpose(1, 2) for gr in grads], dim=2)  # (B, N, 5, H, D)
    want[:, :, 0] = (want[:, :, 0].float() * 0.125).bfloat16()        # gradient of the unscaled queries
    assert torch.equal(gp.view(B, N, 5, H, D), want)
    # and against the oracle
    inp = SimplicialInputs(q=parts[0].float(), k1=parts[1].float(), v1=parts[2].float(), k2=parts[3].float(),
                           v2=parts[4].float(), query_valid=valid, pair_key_valid=valid, pair_valid=pair_valid)  # fmt: skip
    go = grad_out.view(B, N, H, D).transpose(1, 2).float()
    ref_out, ref_grads = simplicial_forward_backward(inp, go)
    tol = bf16_allowance(inp, go, ref_out, ref_grads)
    assert_rel(y.float().cpu(), ref_out, tol["out"], "out")
    largest = max(float(ref_grads[name].abs().max()) for name in NAMES)
    for name, gr in zip(NAMES, grads):  # (a lone token has dq = dk = 0 exactly: judge zeros on the scale of the others)
        err = float((gr.float().cpu() - ref_grads[name]).abs().max())
        assert err <= max(tol[name] * float(ref_grads[name].abs().max()), 1e-2 * largest), f"d{name}: {err}"
