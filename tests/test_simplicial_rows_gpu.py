"""Row-packed tensor-core simplicial kernels (the default for bf16, head_dim 64, at most 192 tokens) against
the CPU oracle: every packing regime (one query range with several first keys per step, several ranges, two
key slabs), masks with holes on queries, keys and pairs, and the benchmark batch at its full size.

Tolerance: bf16 results within 2e-2 of the oracle's largest value, or no worse than the error the reference's
own bf16 torch path makes against its fp32 core on the same inputs (src/matterformer/models/
simplicial_attention.py:251-297), whichever is larger (conftest.bf16_allowance)."""
import pytest
import torch

import matterformer_b200 as mfb
from matterformer_b200 import _lib, synthetic
from matterformer_b200 import simplicial as simplicial_mod
from conftest import bf16_allowance
from oracle.simplicial_ref import SimplicialInputs, simplicial_forward, simplicial_forward_backward

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NAMES = ("q", "k1", "v1", "k2", "v2")


def _case(B, H, N, seed, *, scale=1 / 8.0, lo=None, hi=None, pair_holes=False, key_holes=False, query_holes=False):
    g = torch.Generator().manual_seed(seed)
    t = {n: (torch.randn(B, H, N, 64, generator=g) * scale).bfloat16().float() for n in NAMES}
    go = torch.randn(B, H, N, 64, generator=g).bfloat16().float()
    n_valid = torch.randint(lo if lo is not None else max(1, N // 2), (hi if hi is not None else N) + 1, (B,), generator=g)
    valid = torch.arange(N)[None, :] < n_valid[:, None]
    kv = valid & (torch.rand(B, N, generator=g) > 0.2) if key_holes else valid
    qv = valid & (torch.rand(B, N, generator=g) > 0.2) if query_holes else valid
    pv = (torch.rand(B, N, N, generator=g) > 0.4) if pair_holes else None
    return SimplicialInputs(**t, query_valid=qv, pair_key_valid=kv, pair_valid=pv), go


def _run(inp, go, backend):
    prev = mfb.set_backend(backend)
    try:
        t = [getattr(inp, n).to(DEV, torch.bfloat16).requires_grad_(True) for n in NAMES]
        qv, kv = inp.query_valid.to(DEV), inp.pair_key_valid.to(DEV)
        pv = inp.pair_valid.to(DEV) if inp.pair_valid is not None else None
        out, lse, out32 = mfb.cuda_simplicial_attention_forward(*[x.detach() for x in t], query_valid=qv,
                                                                pair_key_valid=kv, pair_valid=pv)  # fmt: skip
        y = mfb.simplicial_attention_cuda(*t, query_valid=qv, pair_key_valid=kv, pair_valid=pv)
        grads = torch.autograd.grad(y, t, go.to(DEV, torch.bfloat16))
        torch.cuda.synchronize()
        assert simplicial_mod.device_status() == 0
        return out32.cpu(), lse.cpu(), {n: g.float().cpu() for n, g in zip(NAMES, grads)}
    finally:
        mfb.set_backend(prev)


def _rel(a, b, floor=1e-30):
    return (a - b).abs().max().item() / max(b.abs().max().item(), floor)


def _check(inp, go, backend="tcgen05"):
    out_ref, g_ref = simplicial_forward_backward(inp, go)
    _, lse_ref = simplicial_forward(inp, return_lse=True)
    allow = bf16_allowance(inp, go, out_ref, g_ref)
    out, lse, grads = _run(inp, go, backend)
    assert _rel(out, out_ref) <= allow["out"], f"out: {_rel(out, out_ref):.3e} > {allow['out']:.3e}"
    torch.testing.assert_close(lse, lse_ref, atol=3e-2, rtol=1e-2)
    # a gradient that is zero in exact arithmetic (one visible pair: dS = 0) is judged on the scale of the others
    floor = 1e-2 * max(g.abs().max().item() for g in g_ref.values())
    for n in NAMES:
        err = _rel(grads[n], g_ref[n], floor)
        assert err <= allow[n], f"d{n}: {err:.3e} > {allow[n]:.3e}"
    # exact zeros where the oracle has exact zeros (padded queries, keys that take part in no pair)
    dead_q = ~inp.query_valid[:, None, :].expand_as(out[..., 0])
    assert out[dead_q].abs().max() == 0 if dead_q.any() else True
    assert grads["q"][dead_q].abs().max() == 0 if dead_q.any() else True
    dead_k = ~inp.pair_key_valid[:, None, :].expand_as(out[..., 0])
    for n in ("k1", "v1", "k2", "v2"):
        assert grads[n][dead_k].abs().max() == 0 if dead_k.any() else True


# (N, lo, hi): sizes chosen so that the plan has 1, 2, 3, ... first keys per step, one or several query ranges,
# and one or two key slabs (more than 128 keys)
SIZES = [(1, 1, 1), (5, 3, 5), (29, 9, 29), (32, 30, 32), (40, 33, 40), (64, 50, 64), (72, 65, 72), (100, 90, 100),
         (128, 120, 128), (144, 129, 144), (160, 150, 160), (192, 170, 192), (192, 20, 181)]  # fmt: skip


@pytest.mark.parametrize("N,lo,hi", SIZES)
def test_rows_kernels_match_oracle(N, lo, hi):
    inp, go = _case(3, 2, N, seed=7000 + N + lo, lo=lo, hi=hi)
    _check(inp, go)


@pytest.mark.parametrize("N,lo,hi", [(29, 9, 29), (70, 40, 70), (150, 135, 150), (192, 160, 192)])
@pytest.mark.parametrize("holes", ["pair", "key", "query", "all"])
def test_rows_kernels_with_mask_holes(N, lo, hi, holes):
    inp, go = _case(2, 2, N, seed=8000 + N, lo=lo, hi=hi, scale=0.5 if N <= 70 else 1 / 8.0,
                    pair_holes=holes in ("pair", "all"), key_holes=holes in ("key", "all"),
                    query_holes=holes in ("query", "all"))  # fmt: skip
    _check(inp, go)


def test_rows_kernels_peaked_softmax():
    """Scaled-up queries make the softmax sharp: the running maximum moves and rows of one query that sit in
    different groups end with different maxima, which the final merge has to reconcile."""
    inp, go = _case(1, 2, 150, seed=5, lo=140, pair_holes=True)
    inp.q = (inp.q * 48.0).bfloat16().float()
    _check(inp, go)


def test_rows_kernels_many_heads_small_molecules():
    """The trunk's shape: at most 29 tokens, 8 heads, four or more first keys per step."""
    inp, go = _case(16, 8, 29, seed=11, lo=9, hi=29, scale=0.5, pair_holes=True)
    _check(inp, go)


def test_rows_and_tile_kernels_agree():
    """Two independent tensor-core formulations of the same problem."""
    inp, go = _case(4, 4, 181, seed=21, lo=100, hi=181)
    a = _run(inp, go, "tcgen05")
    b = _run(inp, go, "tcgen05_tiles")
    assert _rel(a[0], b[0]) <= 1e-2
    for n in NAMES:
        assert _rel(a[2][n], b[2][n]) <= 2e-2


def test_rows_kernels_deterministic():
    inp, go = _case(3, 2, 170, seed=31, lo=100, hi=170, pair_holes=True)
    a = _run(inp, go, "tcgen05")
    b = _run(inp, go, "tcgen05")
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    for n in NAMES:
        assert torch.equal(a[2][n], b[2][n])


def test_benchmark_batch_backward_matches_oracle():
    """The launch the benchmark times (B=64, N=192, H=8, D=64, atoms uniform in [20,181]): forward and all five
    gradients of three molecules (small, medium, more than 128 atoms) out of the full batch against the oracle."""
    t = synthetic.config2(seed=0)
    n = t["num_atoms"]
    order = torch.argsort(n)
    pick = [int(order[2]), int(order[len(order) // 2]), int(order[-2])]
    assert n[pick[-1]] > 128
    x = [t[k].to(DEV).requires_grad_(True) for k in NAMES]
    valid = t["valid"].to(DEV)
    y = mfb.simplicial_attention_cuda(*x, query_valid=valid, pair_key_valid=valid)
    grads = torch.autograd.grad(y, x, t["grad_out"].to(DEV))
    torch.cuda.synchronize()
    assert simplicial_mod.device_status() == 0
    inp = SimplicialInputs(**{k: t[k][pick].float() for k in NAMES}, query_valid=t["valid"][pick],
                           pair_key_valid=t["valid"][pick])  # fmt: skip
    out_ref, g_ref = simplicial_forward_backward(inp, t["grad_out"][pick].float())
    assert _rel(y[pick].float().cpu(), out_ref) <= 2e-2
    for k, g in zip(NAMES, grads):
        assert _rel(g[pick].float().cpu(), g_ref[k]) <= 2e-2, k
        pad = ~t["valid"][:, None, :].expand(-1, 8, -1)
        assert g.cpu()[pad].abs().max() == 0


def test_row_plan_matches_what_the_kernel_does():
    """The exported plan is the one the kernels evaluate: a molecule whose plan has several ranges and groups
    gives the same bits alone and inside a batch of differently sized molecules."""
    assert _lib.simplicial_row_plan(150, 150)[0] > 1
    inp, go = _case(5, 2, 192, seed=41, lo=30, hi=190)
    out, _, grads = _run(inp, go, "tcgen05")
    one = SimplicialInputs(**{n: getattr(inp, n)[2:3] for n in NAMES}, query_valid=inp.query_valid[2:3],
                           pair_key_valid=inp.pair_key_valid[2:3])  # fmt: skip
    o1, _, g1 = _run(one, go[2:3], "tcgen05")
    assert torch.equal(o1, out[2:3])
    for n in NAMES:
        assert torch.equal(g1[n], grads[n][2:3])
