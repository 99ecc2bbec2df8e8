#!/usr/bin/env python
"""Benchmark of the attention hot path.

Headline workload (always measured, ``metric`` / ``value`` / ``config.workload`` of the JSON line): 2-simplicial
attention forward + backward in bf16 on synthetic drug-like molecules -- B=64, N_max=192, atoms uniform in
[20,181], H=8, D=64, inputs N(0,1)/8.  One step = one forward and one backward pass over the batch through the
C-ABI library.  ``value`` counts the algorithmic FLOPs on valid atoms only, 14*D*H*sum_b n_b^3 (forward 4,
backward 10; recomputation is not counted).  With N > 1 every rank runs the same seeded batch (replicas: the
kernel workload has no exchange step; NCCL carries the barrier and the max-over-ranks of the device time).

Unless ``--no-extra`` is given the line also carries a compact ``workloads`` object with one short timed pass
each of the other operators of the path -- radius block-sparse attention, local-window attention, periodic kNN --
and of the data-parallel trunk step (global batch 1024 split over the ranks, NCCL gradient all-reduce), each with
its roofline fraction, CPU baseline (rank 0, N = 1 only) and end-to-end figure from host buffers.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference          # the reference's own CPU path of the headline workload
    python bench.py --impl reference-triton   # the reference's own Triton kernels on this GPU (kernel to beat)
    python bench.py --workload radius|local|knn|trunk   # one of the other workloads as the main line
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

NAMES = ("q", "k1", "v1", "k2", "v2")
METRIC = "2-simplicial attn fwd+bwd TFLOP/s"
L2_FLUSH_BYTES = 512 << 20
# Kernels this library launches per forward + backward pass of the headline workload (row-packed path): forward =
# extents, launch order, main; backward = extents, launch order, delta, main, finalize.
SIMPLICIAL_LAUNCHES_PER_STEP = 3 + 5
# DRAM bytes (read + written) of ONE launch of the backward kernel on the headline workload, from an ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum); None when no capture of the current kernel exists.
BWD_KERNEL_DRAM_BYTES = 67_346_432  # 45 445 632 read + 21 900 800 written, captured on this workload


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"tflops": float(d["bf16_tflops"]), "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")  # fmt: skip

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)  # fmt: skip
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}  # fmt: skip


def dist_setup():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    return world, rank, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def _reduce(x: float, world: int, dev, op: str) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
    return float(t.item())


def max_over_ranks(x, world, dev):
    return _reduce(x, world, dev, "max")


def sum_over_ranks(x, world, dev):
    return _reduce(x, world, dev, "sum")


def spread(ms: list) -> dict:
    """Median and 10th / 90th percentile of per-step device times."""
    s = sorted(ms)
    pick = lambda f: s[min(len(s) - 1, int(f * len(s)))]  # noqa: E731
    return {"steps": len(s), "median_ms": statistics.median(s), "p10_ms": pick(0.10), "p90_ms": pick(0.90)}


def timed_steps(step, flush, n: int) -> list:
    """Per-step CUDA-event times of ``n`` steps with an L2 flush (outside the events) before each."""
    evs = []
    for _ in range(n):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in evs]


# --------------------------------------------------------------------------------------------
# CPU baselines (rank 0 only): the reference's own torch code when it is installed under baseline/_ref,
# else the restatements of oracle/
# --------------------------------------------------------------------------------------------
def cpu_simplicial(sample_molecules: int, steps: int, warmup: int, seed: int = 0) -> dict:
    """Forward + backward of the dense torch path (fp32, all host threads) on the first ``sample_molecules``
    molecules of the benchmark batch."""
    from matterformer_b200 import synthetic
    from oracle import reference_cpu

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    t = synthetic.config2(seed=seed)
    sel = slice(0, sample_molecules)
    flops = synthetic.simplicial_flops(t["num_atoms"][sel], 8, 64)["total"]
    if reference_cpu.available():
        kind = "reference"
        tensors = {n: t[n][sel] for n in NAMES}
        run = lambda: reference_cpu.simplicial_forward_backward(tensors, t["valid"][sel], t["grad_out"][sel], 128)  # noqa: E731
        what = "the reference's simplicial_attention_torch_from_projected (chunk_size 128) under autograd"
    else:
        from oracle.simplicial_ref import SimplicialInputs, simplicial_forward_backward

        kind = "port"
        inp = SimplicialInputs(**{n: t[n][sel].float() for n in NAMES}, query_valid=t["valid"][sel],
                               pair_key_valid=t["valid"][sel])  # fmt: skip
        go = t["grad_out"][sel].float()
        run = lambda: simplicial_forward_backward(inp, go)  # noqa: E731
        what = "oracle port of the reference torch path"
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        run()
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    return {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": kind,
            "sample": f"first {sample_molecules} of the 64 molecules (atoms {t['num_atoms'][sel].tolist()}), fp32, {what}, "
                      f"{len(times)} timed passes, {sec:.2f} s per pass",
            "ms_per_step": sec * 1e3}  # fmt: skip


def cpu_sparse(workload: str) -> dict:
    """CPU baseline of radius / local attention (fwd+bwd of dense masked SDPA per cell) or of the kNN search."""
    from matterformer_b200 import synthetic
    from oracle import geom_ref, reference_cpu, sparse_ref

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    if workload == "knn":
        t = synthetic.config4(seed=0, with_qkv=False)
        cells = 4
        cell = sparse_ref.lattice_to_cell(t["lattice"][:cells])
        geom_ref.build()
        geom_ref.set_threads(cores)
        geom_ref.knn_topk(t["pos"][:1], cell[:1], t["num_atoms"][:1], 16)
        t0 = time.perf_counter()
        geom_ref.knn_topk(t["pos"][:cells], cell, t["num_atoms"][:cells], 16)
        sec = time.perf_counter() - t0
        pts = cells * t["pos"].shape[1]
        return {"value": pts / sec, "unit": "points/s", "cores": cores, "kind": "port",
                "sample": f"{cells} of 32 cells, C restatement of the adapter distances + (d2, index) selection, all pairs "
                          f"x 27 images, {cores} threads, {sec:.2f} s"}  # fmt: skip
    if workload == "radius":
        t = synthetic.config3(seed=0, batch=1)
        if reference_cpu.available():
            kind = "reference"
            run = lambda: reference_cpu.periodic_masked_attention(t["pos"], t["lattice"], t["q"], t["k"], t["v"], t["cutoff"],
                                                                  t["grad_out"])  # noqa: E731
            what = "the reference's PeriodicGeometryAdapter + masked scaled_dot_product_attention"
        else:
            kind = "port"

            def run():
                vis = sparse_ref.radius_visible(t["pos"], t["lattice"], t["num_atoms"], t["cutoff"])
                q, k, v = (t[n].float().requires_grad_(True) for n in ("q", "k", "v"))
                out = sparse_ref.masked_attention(q, k, v, vis)
                torch.autograd.grad(out, (q, k, v), t["grad_out"].float())

            what = "oracle port of adapter + masked SDPA"
        n_atoms = t["pos"].shape[1]
    else:
        t = synthetic.config4(seed=0, batch=1)
        kind = "port"  # the reference has no band-mask operator: dense SDPA with the band as additive mask

        def run():
            vis = sparse_ref.band_visible(t["q"].shape[2], t["num_atoms"], 64)
            q, k, v = (t[n].float().requires_grad_(True) for n in ("q", "k_", "v"))
            out = sparse_ref.masked_attention(q, k, v, vis)
            torch.autograd.grad(out, (q, k, v), t["grad_out"].float())

        what = "dense masked scaled_dot_product_attention with the band as additive mask (the reference's call)"
        n_atoms = t["q"].shape[2]
    run()
    t0 = time.perf_counter()
    run()
    sec = time.perf_counter() - t0
    return {"value": n_atoms / sec, "unit": "atoms/s", "cores": cores, "kind": kind,
            "sample": f"1 cell of {n_atoms} atoms, fwd+bwd in fp32, {what}, {sec:.2f} s"}  # fmt: skip


def cpu_trunk(batch: int = 64) -> dict:
    """Reduced-batch EDM step of the 12-layer d=512 alternating trunk on the host cores (fp32)."""
    from matterformer_b200 import synthetic
    from oracle import reference_cpu

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    b = synthetic.config5_batch(batch, seed=0)
    b.pop("num_atoms")
    if reference_cpu.available():
        kind, what = "reference", "QM9EDMModel with MHA blocks swapped into the even slots + EDMPreconditioner + EDMLoss"
        net, loss_fn = reference_cpu.build_edm_net()
        step = lambda: reference_cpu.edm_step(net, loss_fn, b)  # noqa: E731
    else:
        from matterformer_b200.dp import build_edm_net
        from matterformer_b200.trunk import EDMLoss

        kind, what = "port", "this repository's mirror of the trunk with the torch attention paths"
        net = build_edm_net(simplicial_impl="torch")
        loss_fn = EDMLoss(sigma_data=1.0)

        def step():
            loss, _ = loss_fn(net, b["atom_types"], b["coords"], b["pad_mask"])
            loss.backward()
            net.zero_grad(set_to_none=True)

    step()
    t0 = time.perf_counter()
    step()
    sec = time.perf_counter() - t0
    return {"value": batch / sec, "unit": "molecules/s", "cores": cores, "kind": kind,
            "sample": f"batch {batch} (of 1024), fp32 forward + backward, {what}, {sec:.2f} s per step"}  # fmt: skip


def run_reference(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    steps = max(1, min(args.steps, 3))
    res = cpu_simplicial(sample_molecules=4, steps=steps, warmup=1)
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": 1, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "simplicial_fwd_bwd_B64_N192_H8_D64 (bounded sample)", "l2": "cpu"},
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


def reference_triton(steps: int = 3, inputs: dict = None, bias=None) -> dict:
    """The reference's own Triton kernels (triton_simplicial_attention_forward / _backward,
    src/matterformer/models/triton_simplicial_attention.py:790-926, 929-1204) on this GPU: on the benchmark batch, or
    on ``inputs`` (a dict like synthetic.simplicial_inputs returns) with the factorized ``bias`` (u, v_bias, w, gate)."""
    from matterformer_b200 import synthetic
    from oracle import reference_cpu

    if not reference_cpu.available():
        return {"unavailable": "the reference is not installed under baseline/_ref"}
    try:
        T = reference_cpu._import("matterformer.models.triton_simplicial_attention")
        if not T.TRITON_AVAILABLE:
            return {"unavailable": "triton is not importable on this machine"}
        t = synthetic.config2(seed=0) if inputs is None else inputs
        x = [t[n].cuda() for n in NAMES]
        valid, go = t["valid"].cuda(), t["grad_out"].cuda()
        none10 = dict(u=None, v_bias=None, w=None, gate=None, angle_left=None, angle_right=None, angle_gate=None,
                      message_left=None, message_right=None, message_basis=None)  # fmt: skip
        no_grads = {k: False for k in ("need_du", "need_dv_bias", "need_dw", "need_dgate", "need_dangle_left",
                                       "need_dangle_right", "need_dangle_gate", "need_dmessage_left",
                                       "need_dmessage_right", "need_dmessage_basis")}  # fmt: skip
        if bias is not None:
            none10.update(u=bias[0].detach(), v_bias=bias[1].detach(), w=bias[2].detach(), gate=bias[3].detach())
            no_grads.update(need_du=True, need_dv_bias=True, need_dw=True, need_dgate=True)
        fwd = lambda: T.triton_simplicial_attention_forward(*x, query_valid=valid, pair_key_valid=valid, pair_valid=None,
                                                            precision="bf16_tc", **none10)  # noqa: E731
        out, lse, out32 = fwd()
        bwd = lambda: T.triton_simplicial_attention_backward(go, *x, out32, lse, query_valid=valid, pair_key_valid=valid,
                                                             pair_valid=None, precision="bf16_tc", **no_grads, **none10)  # noqa: E731
        bwd()
        torch.cuda.synchronize()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        for _ in range(steps):
            fwd()
        e[1].record()
        for _ in range(steps):
            bwd()
        e[2].record()
        torch.cuda.synchronize()
        f_ms, b_ms = e[0].elapsed_time(e[1]) / steps, e[1].elapsed_time(e[2]) / steps
        fl = synthetic.simplicial_flops(t["num_atoms"], x[0].shape[1], x[0].shape[3])
        return {"value": fl["total"] / (f_ms + b_ms) / 1e9, "unit": "TFLOP/s", "fwd_ms": f_ms, "bwd_ms": b_ms,
                "steps": steps, "what": "the reference's Triton forward + backward kernels, bf16_tc, same batch, CUDA events"}  # fmt: skip
    except Exception as ex:  # compile or launch failure of code that is not ours: report, do not retry
        return {"unavailable": f"{type(ex).__name__}: {str(ex)[:200]}"}


# --------------------------------------------------------------------------------------------
# headline workload
# --------------------------------------------------------------------------------------------
def copy_floor_ms(host_in, host_out, dev, steps: int, world: int) -> float:
    """Plain pinned host->device + device->host copies of one step's bytes on two streams, all ranks at once."""
    d_in = [torch.empty(h.shape, dtype=h.dtype, device=dev) for h in host_in]
    d_out = [torch.empty(h.shape, dtype=h.dtype, device=dev) for h in host_out]
    s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    s1.wait_event(e0)
    s2.wait_event(e0)
    for _ in range(steps):
        with torch.cuda.stream(s1):
            for d, h in zip(d_in, host_in):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s2):
            for h, d in zip(host_out, d_out):
                h.copy_(d, non_blocking=True)
    torch.cuda.current_stream().wait_stream(s1)
    torch.cuda.current_stream().wait_stream(s2)
    e1.record()
    torch.cuda.synchronize()
    return max_over_ranks(e0.elapsed_time(e1), world, dev) / steps


def run_simplicial(args, world, rank, local) -> dict:
    import matterformer_b200 as mfb
    from matterformer_b200 import _lib, synthetic

    dev = torch.device(f"cuda:{local}")
    t = synthetic.config2(seed=0, batch=args.batch)
    x = [t[n].to(dev) for n in NAMES]
    valid = t["valid"].to(dev)
    go = t["grad_out"].to(dev)
    fl = synthetic.simplicial_flops(t["num_atoms"], 8, 64)
    flush = torch.empty(L2_FLUSH_BYTES, device=dev, dtype=torch.uint8)

    def step():
        out, lse, out32 = mfb.cuda_simplicial_attention_forward(*x, query_valid=valid, pair_key_valid=valid,
                                                                pair_valid=None)  # fmt: skip
        return mfb.cuda_simplicial_attention_backward(go, *x, out32, lse, query_valid=valid, pair_key_valid=valid,
                                                      pair_valid=None)  # fmt: skip

    for _ in range(args.warmup):
        flush.zero_()
        step()
    barrier(world)
    sampler = ClockSampler(local)
    sampler.start()
    _lib.profile_enable(True)
    per_step = timed_steps(step, flush, args.steps)  # exactly K steps, L2 flushed before each, outside the events
    barrier(world)
    _lib.profile_enable(False)
    fwd_ms, fwd_n = _lib.profile_read(0)
    bwd_ms, bwd_n = _lib.profile_read(1)
    more = timed_steps(step, flush, max(0, 100 - args.steps))  # at least 100 timed steps for the spread
    barrier(world)
    clocks = sampler.stop()
    status = mfb.simplicial.device_status()
    if status != 0:
        raise SystemExit(f"the tensor-core kernels reported device status {status}")
    total_ms = max_over_ranks(sum(per_step), world, dev)
    total_flops = sum_over_ranks(fl["total"], world, dev)
    value = total_flops * args.steps / (total_ms * 1e-3) / 1e12

    # ---- end to end through the public API with host buffers (pinned), copies inside the timed region
    host_in = [t[n].pin_memory() for n in NAMES] + [t["grad_out"].pin_memory()]
    host_out = [torch.empty_like(t["q"]).pin_memory() for _ in range(6)]
    h2d = sum(h.numel() * h.element_size() for h in host_in)
    d2h = sum(h.numel() * h.element_size() for h in host_out)
    pipe = mfb.HostPipelinedSimplicial(dev, query_valid=valid, pair_key_valid=valid)
    for _ in range(max(args.warmup, 3)):
        pipe.submit(host_in, host_out)
    pipe.finish()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(3, min(args.steps, 10))
    e0.record(pipe.s_in)
    for _ in range(e2e_steps):
        pipe.submit(host_in, host_out)
    e1.record(pipe.s_out)
    pipe.finish()
    barrier(world)
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), world, dev)
    e2e_value = total_flops * e2e_steps / (e2e_ms * 1e-3) / 1e12
    floor = copy_floor_ms(host_in, host_out, dev, e2e_steps, world)

    peaks = measured_peaks()
    bwd_tflops = fl["bwd"] * bwd_n / (bwd_ms * 1e-3) / 1e12 if bwd_ms > 0 else None
    fwd_tflops = fl["fwd"] * fwd_n / (fwd_ms * 1e-3) / 1e12 if fwd_ms > 0 else None
    return {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"simplicial_fwd_bwd_B{args.batch}_N192_H8_D64", "atoms": "uniform[20,181]",
                   "batch_per_gpu": args.batch, "multi_gpu": "replicas: the same seeded batch on every rank",
                   "l2": "flushed between timed steps (512 MiB write)", "flops": "valid atoms only, 14*D*H*sum n^3",
                   "pct_of_measured_bf16_peak": 100.0 * value / world / peaks["tflops"]},
        "stats": spread(per_step + more),
        "roofline": {"bound": "tensor", "achieved": bwd_tflops, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": (bwd_tflops / peaks["tflops"]) if bwd_tflops else None, "traffic": BWD_KERNEL_DRAM_BYTES,
                     "kernel": "simplicial_rows_bwd_kernel", "peak_source": peaks["source"] + " (burst)",
                     "kernel_ms": bwd_ms / max(bwd_n, 1), "fwd_kernel": "simplicial_rows_fwd_kernel",
                     "fwd_kernel_tflops": fwd_tflops, "fwd_kernel_ms": fwd_ms / max(fwd_n, 1),
                     "fwd_frac": (fwd_tflops / peaks["tflops"]) if fwd_tflops else None},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms / e2e_steps, "copy_floor_ms": floor,
                # floor of a pipelined step = the slower of its copies and its kernels
                "over_floor": (e2e_ms / e2e_steps) / max(floor, total_ms / args.steps)},
        "gpu_launches": SIMPLICIAL_LAUNCHES_PER_STEP * args.steps,
        "clocks": clocks,
    }  # fmt: skip


# --------------------------------------------------------------------------------------------
# radius / local / kNN
# --------------------------------------------------------------------------------------------
def run_sparse(workload: str, steps: int, warmup: int, world, rank, local, with_cpu: bool) -> dict:
    """Radius block-sparse attention (fwd+bwd), local-window attention (fwd+bwd) or the periodic kNN search."""
    import matterformer_b200 as mfb
    from matterformer_b200 import synthetic

    dev = torch.device(f"cuda:{local}")
    peaks = measured_peaks()
    flush = torch.empty(L2_FLUSH_BYTES, device=dev, dtype=torch.uint8)
    extra = {}
    if workload == "knn":
        t = synthetic.config4(seed=0, with_qkv=False)
        host_in = [t["pos"].pin_memory()]
        pos, cell, na = t["pos"].to(dev), mfb.lattice_latent_to_cell(t["lattice"]).to(dev), t["num_atoms"].to(dev)
        step = lambda: mfb.knn_topk(pos, cell, na, k=16)  # noqa: E731
        units = pos.shape[0] * pos.shape[1]
        bytes_alg = units * (12 + 16 * 4 + 16 * 4)
        metric, unit, name, launches = "periodic kNN k=16 points/s", "points/s", "knn_B32_N4096_k16", 7
        host_out = [torch.empty(*pos.shape[:2], 16, dtype=torch.int32).pin_memory(),
                    torch.empty(*pos.shape[:2], 16, dtype=torch.float32).pin_memory()]  # fmt: skip

        def e2e_step():
            idx, d2 = mfb.knn_topk(host_in[0].to(dev, non_blocking=True), cell, na, k=16)
            host_out[0].copy_(idx, non_blocking=True)
            host_out[1].copy_(d2, non_blocking=True)

    else:
        if workload == "radius":
            t = synthetic.config3(seed=0)
            pos_d, lat_d, na = t["pos"].to(dev), t["lattice"].to(dev), t["num_atoms"].to(dev)
            blocks = mfb.build_radius_blocks(pos_d, lat_d, na, t["cutoff"])
            q, k, v = (t[n].to(dev).requires_grad_(True) for n in ("q", "k", "v"))
            fwd = lambda: mfb.radius_block_sparse_attention(q, k, v, blocks)  # noqa: E731
            name = "radius_attn_fwd_bwd_B16_N1024_H8_D64_cutoff6"
            kn = "k"
            active = int(blocks.block_count.sum())
            T = blocks.block_count.shape[1]
            extra["block_density"] = active / (blocks.block_count.shape[0] * T * T)
            forced = mfb.sparse._SPARSE_BACKEND
            extra["kernels"] = {"auto": "tcgen05, 128-row tiles", "tcgen05": "tcgen05, 128-row tiles",
                                "mma": "mma.sync, 32-row tiles"}[forced]  # fmt: skip
            lut = torch.tensor([bin(i).count("1") for i in range(256)], dtype=torch.int64, device=dev)
            live = (torch.arange(T, device=dev)[None, None, :] < blocks.block_count[:, :, None])[..., None]  # listed blocks
            words = (blocks.block_mask * live).contiguous().view(torch.uint8).long()
            pairs = int(lut[words].sum())  # atom pairs within the cutoff (bits of the per-block masks)
        else:
            t = synthetic.config4(seed=0)
            q, k, v = (t[n].to(dev).requires_grad_(True) for n in ("q", "k_", "v"))
            na = t["num_atoms"].to(dev)
            fwd = lambda: mfb.local_window_attention(q, k, v, na, window=64)  # noqa: E731
            name = "local_attn_fwd_bwd_B32_N4096_H8_D64_w64"
            kn = "k_"
            pairs = None
            extra["kernels"] = "tcgen05, 128-row tiles" if mfb.sparse._SPARSE_BACKEND == "tcgen05" else "mma.sync, 32-row tiles"
        go = t["grad_out"].to(dev)

        def step():
            out = fwd()
            return torch.autograd.grad(out, [q, k, v], go)

        units = q.shape[0] * q.shape[2]
        nbytes = q.numel() * 2
        bytes_alg = 4 * nbytes + 8 * nbytes  # fwd: q,k,v,o; bwd: q,k,v,o,do + dq,dk,dv
        metric, unit, launches = f"{workload} attention fwd+bwd atoms/s", "atoms/s", 3  # forward, dq (+ delta), dk+dv
        host_in = [t[n].pin_memory() for n in ("q", kn, "v", "grad_out")]
        host_out = [torch.empty_like(t["q"]).pin_memory() for _ in range(4)]

        def e2e_step():
            qd, kd, vd, gd = (h.to(dev, non_blocking=True) for h in host_in)
            qd, kd, vd = (x.requires_grad_(True) for x in (qd, kd, vd))
            if workload == "radius":
                out = mfb.radius_block_sparse_attention(qd, kd, vd, blocks)
            else:
                out = mfb.local_window_attention(qd, kd, vd, na, window=64)
            grads = torch.autograd.grad(out, [qd, kd, vd], gd)
            for h, g in zip(host_out, (out.detach(), *grads)):
                h.copy_(g, non_blocking=True)

    for _ in range(warmup):
        flush.zero_()
        step()
    barrier(world)
    sampler = ClockSampler(local)
    sampler.start()
    per_step = timed_steps(step, flush, steps)
    barrier(world)
    clocks = sampler.stop()
    ms = max_over_ranks(sum(per_step), world, dev)
    value = units * world * steps / (ms * 1e-3)
    gbs = bytes_alg * steps / (ms * 1e-3) / 1e9
    # end to end from pinned host buffers
    e2e_step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_e2e = max(3, min(steps, 10))
    e0.record()
    for _ in range(n_e2e):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), world, dev) / n_e2e
    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if workload == "knn" else "bf16", "data": "synthetic",
        "config": {"workload": name, "l2": "flushed between timed steps (512 MiB write)", **extra},
        "stats": spread(per_step),
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "traffic": None, "peak_source": peaks["source"],
                     "note": "whole step (all kernels of the op) over algorithmic bytes"},
        "e2e": {"value": units * world / (e2e_ms * 1e-3), "unit": unit, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": sum(h.numel() * h.element_size() for h in host_in),
                "d2h_bytes_per_step": sum(h.numel() * h.element_size() for h in host_out)},
        "gpu_launches": launches * steps, "clocks": clocks,
    }  # fmt: skip
    if workload == "knn":
        n = pos.shape[1]
        line["roofline"]["pair_evaluations_per_s"] = {
            "all_pairs_27_images_equivalent": pos.shape[0] * n * n * 27 * steps / (ms * 1e-3),
            "note": "what the reference's adapter evaluates for the same answer; the real bound of this kernel is "
                    "fp32 distance + selection issue rate (about 1000 warp instructions per query), not HBM"}  # fmt: skip
    if workload == "radius" and pairs is not None:
        flops = 4.0 * 64 * 8 * pairs * 3.5  # QK^T + PV forward, 2.5x that backward, on unmasked pairs only
        tf = flops * steps / (ms * 1e-3) / 1e12
        line["roofline"]["tensor"] = {"achieved": tf, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": tf / peaks["tflops"],
                                      "note": "4*D*H*(pairs within the cutoff)*3.5 FLOPs; at this density the operator is dense "
                                              "masked attention and the tensor roof, not HBM, is the one that binds"}  # fmt: skip
    if with_cpu and rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_sparse(workload)
    return line


def run_bias(steps: int, warmup: int, world, rank, local, shape: str = "small", with_reference_kernels: bool = True) -> dict:
    """2-simplicial attention with the factorized geometry bias (the reference model's default geometry mode,
    models/qm9.py:261), forward + backward on the tcgen05 tile kernels, which add the bias to the logits in fp32 and
    form its four gradients in the backward kernel's element-wise pass.  ``shape`` "small": 256 molecules of 9..29
    atoms, four heads per tile; "config2": the benchmark batch (64 molecules of 128..192 atoms), one head per tile."""
    import matterformer_b200 as mfb
    from matterformer_b200 import synthetic

    dev = torch.device(f"cuda:{local}")
    if shape == "config2":
        t = synthetic.config2(seed=0)
        B, H, N, D = t["q"].shape
    else:
        B, N, H, D = 256, 29, 8, 64
        t = synthetic.simplicial_inputs(B, N, 9, 29, H, D, 1.0 / 8.0, 0, torch.bfloat16)
    g = torch.Generator().manual_seed(1)
    leaves = [t[n].to(dev).requires_grad_(True) for n in ("q", "k1", "v1", "k2", "v2")]
    bias = [(torch.randn(B, H, N, N, generator=g) * 0.5).to(dev).requires_grad_(True) for _ in range(3)]
    bias.append(torch.randn(B, H, N, generator=g).to(dev).requires_grad_(True))
    valid, go = t["valid"].to(dev), t["grad_out"].to(dev)

    def step():
        y = mfb.simplicial_attention_cuda(*leaves, query_valid=valid, pair_key_valid=valid, factorized_bias=tuple(bias))
        return torch.autograd.grad(y, leaves + bias, go)

    flush = torch.empty(L2_FLUSH_BYTES, device=dev, dtype=torch.uint8)
    for _ in range(warmup):
        step()
    barrier(world)
    per_step = timed_steps(step, flush, steps)
    barrier(world)
    ms = max_over_ranks(sum(per_step), world, dev)
    flops = synthetic.simplicial_flops(t["num_atoms"], H, D)["total"]
    peaks = measured_peaks()
    tf = flops * world * steps / (ms * 1e-3) / 1e12
    k2b = reference_triton(steps=3, inputs=t, bias=bias) if (rank == 0 and world == 1 and with_reference_kernels) else None
    return {
        "metric": METRIC, "value": tf, "unit": "TFLOP/s", "ms_per_step": ms / steps, "scaling": "weak", "dtype": "bf16",
        "config": {"workload": f"simplicial_fwd_bwd_factorized_bias_B{B}_N{N}_H{H}_D{D}",
                   "kernels": "tcgen05 tile kernels, %s, bias added in fp32" % ("one head per tile" if shape == "config2"
                                                                                else "four heads per tile"),
                   "gradients": "q, k1, v1, k2, v2, u, v_bias, w, gate", "kernel_to_beat": k2b},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": tf / peaks["tflops"], "peak_source": peaks["source"],
                     "note": "valid FLOPs 14*D*H*sum n^3 over forward + backward"},
        "stats": spread(per_step),
    }  # fmt: skip


# --------------------------------------------------------------------------------------------
# data-parallel trunk
# --------------------------------------------------------------------------------------------
def trunk_flops_per_step(num_atoms: torch.Tensor, d: int = 512, layers: int = 12) -> float:
    """Model FLOPs of one EDM step (forward + backward = 3x forward) on valid tokens only: linear layers
    n*312*d^2, six simplicial cores 4*n^3*d each, six MHA cores 4*n^2*d each, adaLN 12*12*d^2 per molecule."""
    n = num_atoms.double()
    fwd = (n * 312 * d * d + (layers // 2) * 4 * n**3 * d + (layers // 2) * 4 * n**2 * d + 12 * layers * d * d).sum()
    return 3.0 * float(fwd)


def run_trunk(steps: int, warmup: int, world, rank, local, global_batch: int, no_graph: bool, with_cpu: bool) -> dict:
    """Dense-token trunk, EDM denoising step forward + backward + AdamW, data parallel: global batch split evenly over
    the ranks (strong scaling), NCCL all-reduce of the gradients overlapped with backward."""
    from matterformer_b200 import synthetic
    from matterformer_b200.dp import build_edm_net, edm_train_step, shard_batch, wrap_data_parallel
    from matterformer_b200.trunk import EDMLoss

    dev = torch.device(f"cuda:{local}")
    full = synthetic.config5_batch(global_batch, seed=0)
    num_atoms = full.pop("num_atoms")
    host = {k: v.pin_memory() for k, v in shard_batch(full, rank, world).items()}
    batch = {k: v.to(dev) for k, v in host.items()}
    net = build_edm_net(seed=0).to(dev)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):  # DDP built on the stream the step will be captured on
        ddp = wrap_data_parallel(net, dev)
    torch.cuda.current_stream().wait_stream(side)
    opt = torch.optim.AdamW(net.parameters(), lr=1e-4, fused=True, capturable=not no_graph)
    loss_fn = EDMLoss(sigma_data=1.0)
    torch.manual_seed(1234 + rank)
    mode = "eager"
    step = lambda b=None: edm_train_step(ddp, loss_fn, opt, batch if b is None else b)  # noqa: E731
    if not no_graph:
        from matterformer_b200.dp import GraphedTrainStep

        graphed = GraphedTrainStep(ddp, loss_fn, opt, batch, warmup=max(11, warmup))
        step, mode = graphed, "cuda_graph"
    for _ in range(warmup):
        step()
    barrier(world)
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier(world)
    clocks = sampler.stop()
    ms = max_over_ranks(e0.elapsed_time(e1), world, dev)
    value = global_batch * steps / (ms * 1e-3)
    # end to end: the shard comes from pinned host memory every step and the loss is read back
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    e0.record()
    for _ in range(steps):
        if mode == "cuda_graph":
            float(step(host))
        else:
            float(step({k: v.to(dev, non_blocking=True) for k, v in host.items()}))
    e1.record()
    barrier(world)
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), world, dev)
    # the same step without the exchange: what the all-reduce costs on top of the shrinking per-GPU batch
    # (both legs launched eagerly: a graph replay and an eager step are not comparable)
    no_sync_ms = sync_ms = None
    if world > 1:
        def eager_leg(exchange: bool) -> float:
            def one():
                if exchange:
                    edm_train_step(ddp, loss_fn, opt, batch)
                else:
                    with ddp.no_sync():
                        edm_train_step(ddp, loss_fn, opt, batch)

            n = max(3, steps // 2)
            for _ in range(3):
                one()
            barrier(world)
            e0.record()
            for _ in range(n):
                one()
            e1.record()
            barrier(world)
            return max_over_ranks(e0.elapsed_time(e1), world, dev) / n

        no_sync_ms, sync_ms = eager_leg(False), eager_leg(True)
    peaks = measured_peaks()
    tf = trunk_flops_per_step(num_atoms) * steps / (ms * 1e-3) / 1e12
    params = sum(p.numel() for p in net.parameters())
    line = {
        "metric": "trunk EDM step molecules/s", "value": value, "unit": "molecules/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "trunk_edm_step_L12_d512_H8_alternating_mha_simplicial", "global_batch": global_batch,
                   "atoms": "uniform[9,29]", "params": params, "parallelism": f"dp{world}", "launch": mode,
                   "allreduce_bytes_per_step": 4 * params if world > 1 else 0,
                   "eager_ms_per_step_without_allreduce": no_sync_ms, "eager_ms_per_step_with_allreduce": sync_ms,
                   "l2": "working set (weights + optimizer state + activations) exceeds L2"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["tflops"] * world, "unit": "TFLOP/s",
                     "frac": tf / (peaks["tflops"] * world), "traffic": None, "peak_source": peaks["source"],
                     "note": "whole step, model FLOPs on valid tokens / step time / (n_gpus * bf16 peak)"},
        "e2e": {"value": global_batch * steps / (e2e_ms * 1e-3), "unit": "molecules/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / steps},
        "gpu_launches": None, "clocks": clocks,
    }  # fmt: skip
    if with_cpu and rank == 0 and world == 1:
        line["cpu_baseline"] = cpu_trunk()
    return line


def compact(line: dict) -> dict:
    keep = ("metric", "value", "unit", "ms_per_step", "scaling", "dtype", "config", "roofline", "e2e", "cpu_baseline", "stats")
    return {k: line[k] for k in keep if k in line}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-triton"])
    ap.add_argument("--workload", default="simplicial", choices=["simplicial", "radius", "local", "knn", "trunk", "bias", "bias_config2"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="headline workload only: skip the compact passes over the other workloads")
    ap.add_argument("--no-reference-kernels", action="store_true",
                    help="skip the timing of the reference's Triton kernels (kernel_to_beat); for profiler runs")
    ap.add_argument("--no-graph", action="store_true", help="trunk workload: launch the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--batch", type=int, default=64, help="molecules per GPU (simplicial workload; 64 = the benchmark)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the package has no CPU fallback)")
    if args.impl == "reference-triton":
        if int(os.environ.get("RANK", "0")) == 0:
            res = reference_triton(steps=max(1, min(args.steps, 5)))
            print(json.dumps({"impl": "reference-triton", "metric": METRIC, "higher_is_better": True, "n_gpus": 1,
                              "config": {"workload": "simplicial_fwd_bwd_B64_N192_H8_D64"}, **res}), flush=True)  # fmt: skip
        return
    world, rank, local = dist_setup()
    with_cpu = not args.no_cpu_baseline
    if args.workload == "simplicial":
        line = run_simplicial(args, world, rank, local)
        if not args.no_extra:
            extras = {}
            for w in ("radius", "local", "knn"):
                extras[w] = compact(run_sparse(w, 20, 5, world, rank, local, with_cpu))
            extras["simplicial_bias"] = compact(run_bias(20, 5, world, rank, local))
            extras["simplicial_bias_config2"] = compact(run_bias(5, 3, world, rank, local, "config2"))
            extras["trunk"] = compact(run_trunk(10, 3, world, rank, local, 1024, False, with_cpu))
            line["workloads"] = extras
        if rank == 0 and world == 1:
            if with_cpu:
                res = cpu_simplicial(sample_molecules=4, steps=2, warmup=1)
                line["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
            if not args.no_reference_kernels:
                line["kernel_to_beat"] = reference_triton(steps=3)
    elif args.workload == "trunk":
        line = run_trunk(args.steps, args.warmup, world, rank, local, args.batch if args.batch != 64 else 1024,
                         args.no_graph, with_cpu)  # fmt: skip
    elif args.workload in ("bias", "bias_config2"):
        line = run_bias(args.steps, args.warmup, world, rank, local, "config2" if args.workload == "bias_config2" else "small",
                        not args.no_reference_kernels)
    else:
        line = run_sparse(args.workload, args.steps, args.warmup, world, rank, local, with_cpu)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
