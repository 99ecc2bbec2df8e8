"""The drop-in boundary, end to end: the reference's own ``SimplicialAttention`` / 21-argument autograd function
run on this library's kernels after ``install()``, on CUDA, with the shapes and tolerances of the reference's GPU
parity tests (tests/test_simplicial_attention.py:841-896 and :901-1020), checked against the reference's torch
path with its fp32 core.

The reference is taken from ``baseline/_ref`` (``pip install --no-deps --target baseline/_ref <reference>``; the
directory is not part of the source tree but travels with it to the GPU machine).  Without it these tests are
skipped with that reason.  The product package never imports it.
"""
import sys
from pathlib import Path

import pytest
import torch

import matterformer_b200 as mfb
from matterformer_b200 import simplicial as S

pytestmark = pytest.mark.gpu
DEV = "cuda"
REF_DIR = Path(__file__).resolve().parents[1] / "baseline" / "_ref"


@pytest.fixture()
def ref():
    if not (REF_DIR / "matterformer").is_dir():
        pytest.skip(f"the reference is not installed under {REF_DIR} (see the module docstring)")
    sys.path.insert(0, str(REF_DIR))
    try:
        import matterformer.models.simplicial_attention as module
    finally:
        sys.path.remove(str(REF_DIR))
    calls = {"fwd": 0, "bwd": 0}
    fwd, bwd = S.cuda_simplicial_attention_forward, S.cuda_simplicial_attention_backward

    def counted_fwd(*a, **k):
        calls["fwd"] += 1
        return fwd(*a, **k)

    def counted_bwd(*a, **k):
        calls["bwd"] += 1
        return bwd(*a, **k)

    mfb.install(module)
    module.triton_simplicial_attention_forward = counted_fwd
    module.triton_simplicial_attention_backward = counted_bwd
    module._mfb_calls = calls
    try:
        yield module
    finally:
        mfb.uninstall(module)


def _apply(ref, q, k1, v1, k2, v2, mask, *, bias=None, angle=None, message=None, basis=None, precision="ieee_fp32"):
    """ref: _apply_triton_function of the reference's tests (tests/test_simplicial_attention.py:187-241)."""
    e = q.new_empty(0)
    eb = torch.empty(0, device=q.device, dtype=torch.bool)
    u, v, w, gate = (bias.u, bias.v, bias.w, bias.gate) if bias is not None else (e, e, e, e)
    al, ar, ag = (angle.left, angle.right, angle.gate) if angle is not None else (e, e, e)
    ml, mr, mb = (message.left, message.right, basis) if message is not None else (e, e, e)
    return ref._TritonTwoSimplicialAttentionFunction.apply(
        q, k1, v1, k2, v2, mask.query_valid, mask.pair_key_valid, mask.pair_valid if mask.pair_valid is not None else eb,
        u, v, w, gate, al, ar, ag, ml, mr, mb, precision, 2, False)  # fmt: skip


def _leaves(shape, n, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(*shape, generator=g).to(DEV).requires_grad_(True) for _ in range(n)]


def test_no_bias_forward_backward_matches_reference_torch_path(ref):
    """Shapes and tolerance of test_triton_no_bias_forward_backward_matches_torch_cuda."""
    a = _leaves((2, 4, 5, 8), 5, 0)
    b = [t.detach().clone().requires_grad_(True) for t in a]
    pad = torch.tensor([[False, False, False, False, True], [False, False, True, True, True]], device=DEV)
    mask = ref.SimplicialAttentionMask.from_key_padding_mask(pad, batch_size=2, num_tokens=5, device=torch.device(DEV))
    want = ref.simplicial_attention_torch_from_projected(*a, attention_mask=mask, chunk_size=2, fp32_core=True)
    got = _apply(ref, *b, mask)
    assert ref._mfb_calls["fwd"] == 1
    torch.testing.assert_close(got, want, atol=1e-4, rtol=1e-4)
    want.square().mean().backward()
    got.square().mean().backward()
    assert ref._mfb_calls["bwd"] == 1
    for x, y in zip(b, a):
        torch.testing.assert_close(x.grad, y.grad, atol=1e-4, rtol=1e-4)


def test_factorized_angle_and_message_match_reference_torch_path(ref):
    """Shapes and tolerance of test_triton_factorized_angle_and_message_matches_torch_cuda: factorized bias, angle
    residual of rank 5, message residual of rank 3 and a pair mask with holes; all fifteen gradients."""
    B, H, N, D = 1, 2, 7, 8
    a = _leaves((B, H, N, D), 5, 1)
    b = [t.detach().clone().requires_grad_(True) for t in a]
    extra_a = _leaves((B, H, N, N), 3, 2) + _leaves((B, H, N), 1, 3) + _leaves((B, H, N, N, 5), 2, 4) + \
        _leaves((B, H, N), 1, 5) + _leaves((B, H, N, N, 3), 2, 6) + _leaves((H, 3, D), 1, 7)  # fmt: skip
    extra_b = [t.detach().clone().requires_grad_(True) for t in extra_a]

    def pack(e):
        return (ref.SimplicialFactorizedBias(u=e[0], v=e[1], w=e[2], gate=e[3]),
                ref.SimplicialLowRankAngleResidual(left=e[4], right=e[5], gate=e[6]),
                ref.SimplicialLowRankMessageResidual(left=e[7], right=e[8]), e[9])  # fmt: skip

    pad = torch.tensor([[False] * 5 + [True] * 2], device=DEV)
    m0 = ref.SimplicialAttentionMask.from_key_padding_mask(pad, batch_size=B, num_tokens=N, device=torch.device(DEV))
    pv = torch.ones(B, N, N, device=DEV, dtype=torch.bool)
    pv[:, 1, 4] = False
    pv[:, 4, 1] = False
    mask = ref.SimplicialAttentionMask(query_valid=m0.query_valid, pair_key_valid=m0.pair_key_valid, pair_valid=pv)
    fa, aa, ma, ba = pack(extra_a)
    fb, ab, mb_, bb = pack(extra_b)
    want = ref.simplicial_attention_torch_from_projected(*a, attention_mask=mask, factorized_bias=fa, angle_residual=aa,
                                                         message_residual=ma, message_basis=ba, chunk_size=3,
                                                         fp32_core=True)  # fmt: skip
    got = _apply(ref, *b, mask, bias=fb, angle=ab, message=mb_, basis=bb)
    torch.testing.assert_close(got, want, atol=1e-4, rtol=1e-4)
    want.square().mean().backward()
    got.square().mean().backward()
    for x, y in zip(b + extra_b, a + extra_a):
        torch.testing.assert_close(x.grad, y.grad, atol=1e-4, rtol=1e-4)


def test_cancelling_bias_terms_are_summed_in_fp32(ref):
    """u ~ +1000 and v ~ -1000 with gate 1 (the stress input of scripts/diagnose_simplicial_triton_parity.py:80-84):
    a kernel that adds the bias terms in low precision or in another order than the reference
    (tests/test_simplicial_attention.py:299-311) loses the small difference that decides the softmax."""
    B, H, N, D = 1, 2, 9, 16
    a = _leaves((B, H, N, D), 5, 11)
    b = [t.detach().clone().requires_grad_(True) for t in a]
    g = torch.Generator().manual_seed(12)
    u = (1000.0 + torch.randn(B, H, N, N, generator=g)).to(DEV)
    v = (-1000.0 + torch.randn(B, H, N, N, generator=g)).to(DEV)
    w = torch.randn(B, H, N, N, generator=g).to(DEV)
    gate = torch.ones(B, H, N, device=DEV)
    bias = ref.SimplicialFactorizedBias(u=u, v=v, w=w, gate=gate)
    mask = ref.SimplicialAttentionMask.from_key_padding_mask(torch.zeros(B, N, dtype=torch.bool, device=DEV),
                                                             batch_size=B, num_tokens=N, device=torch.device(DEV))  # fmt: skip
    want = ref.simplicial_attention_torch_from_projected(*a, attention_mask=mask, factorized_bias=bias, chunk_size=4,
                                                         fp32_core=True)  # fmt: skip
    got = _apply(ref, *b, mask, bias=bias)
    torch.testing.assert_close(got, want, atol=1e-4, rtol=1e-4)
    want.square().mean().backward()
    got.square().mean().backward()
    for x, y in zip(b, a):
        torch.testing.assert_close(x.grad, y.grad, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("tokens,dim,heads", [(40, 512, 8), (150, 512, 8)])
def test_reference_module_runs_on_the_tensor_core_kernels(ref, tokens, dim, heads):
    """``SimplicialAttention(impl="triton", precision="bf16_tc")`` of the reference under bf16 autocast (how its
    training scripts run it), forward and backward through its projections, against the same module with
    ``impl="torch"`` in fp32.  Outputs and input gradients within 2e-2 of the largest value; parameter gradients
    within the 5e-2 the reference's own bf16 validation allows (scripts/validate_simplicial_attention.py:81-82)."""
    torch.manual_seed(0)
    fast = ref.SimplicialAttention(dim, heads, impl="triton", precision="bf16_tc").to(DEV)
    slow = ref.SimplicialAttention(dim, heads, impl="torch", chunk_size=16).to(DEV)
    slow.load_state_dict(fast.state_dict())
    x = torch.randn(3, tokens, dim, device=DEV)
    n_valid = torch.tensor([tokens, tokens - 7, max(1, tokens // 2)], device=DEV)
    pad = torch.arange(tokens, device=DEV)[None, :] >= n_valid[:, None]
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        ya = fast(xa, key_padding_mask=pad)
    assert fast._last_impl_used == "triton" and ref._mfb_calls["fwd"] == 1
    yb = slow(xb, key_padding_mask=pad)
    keep = (~pad)[..., None].float()
    go = torch.randn_like(yb) * keep
    ya.float().backward(go)
    yb.backward(go)
    assert ref._mfb_calls["bwd"] == 1 and S.device_status() == 0

    def rel(p, q):
        return (p.float() - q).abs().max().item() / q.abs().max().item()

    errs = {"out": rel(ya * keep, yb * keep), "dx": rel(xa.grad * keep, xb.grad * keep)}
    for (name, pa), (_, pb) in zip(fast.named_parameters(), slow.named_parameters()):
        errs[name] = rel(pa.grad, pb.grad)
    assert errs["out"] <= 2e-2 and errs["dx"] <= 2e-2, errs
    assert max(errs.values()) <= 5e-2, errs


def test_limits_of_this_backend_surface_through_the_reference_path(ref):
    """Residual ranks above 32 (the reference's kernel takes 64): ``impl="auto"`` falls back to the torch path,
    ``impl="triton"`` raises with a reason.  batch * heads above 65535 raises a clear error."""
    B, H, N, D, R = 1, 2, 6, 8, 40
    x = torch.randn(B, N, H * D, device=DEV)
    g = torch.Generator().manual_seed(5)
    angle = ref.SimplicialLowRankAngleResidual(left=torch.randn(B, H, N, N, R, generator=g).to(DEV),
                                               right=torch.randn(B, H, N, N, R, generator=g).to(DEV),
                                               gate=torch.randn(B, H, N, generator=g).to(DEV))  # fmt: skip
    auto = ref.SimplicialAttention(H * D, H, impl="auto", precision="ieee_fp32").to(DEV)
    auto(x, angle_residual=angle)
    assert auto._last_impl_used == "torch"
    forced = ref.SimplicialAttention(H * D, H, impl="triton", precision="ieee_fp32").to(DEV)
    with pytest.raises(RuntimeError, match="ranks up to 32"):
        forced(x, angle_residual=angle)
    big = torch.zeros(65536, 1, 1, 8, device=DEV)
    ok = torch.ones(65536, 1, dtype=torch.bool, device=DEV)
    with pytest.raises(ValueError, match="batch\\*heads above 65535"):
        mfb.cuda_simplicial_attention_forward(big, big, big, big, big, query_valid=ok, pair_key_valid=ok, pair_valid=None)
