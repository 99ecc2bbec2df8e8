#!/usr/bin/env python
"""Benchmark of the attention hot path.

Default workload (``--workload simplicial``): 2-simplicial attention forward + backward in bf16 on
synthetic drug-like molecules -- B=64, N_max=192, atoms uniform in [20,181], H=8, D=64, inputs
N(0,1)/8 -- the configuration the headline metric is quoted on.  One step = one forward and one
backward pass over the batch through the C-ABI library.  ``value`` counts the algorithmic FLOPs
on valid atoms only, 14*D*H*sum_b n_b^3 (forward 4, backward 10; recomputation is not counted).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference         # the reference's CPU path (oracle port) on the host cores

With N > 1 every rank runs its own batch of the same shape (different seed): the batch of
structures shards with no data-path collective, so scaling is weak; NCCL is used for the barrier and
the max-over-ranks of the device time only.  Other workloads: ``--workload radius|local|knn``.
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

# DRAM traffic of one launch of the backward kernel on the benchmark workload (bytes read + written), from
# the ncu capture summarised under profiles/; None until that capture exists.
BWD_KERNEL_DRAM_BYTES = 132_152_832  # 46.4 MB read + 85.7 MB written (profiles/simplicial_sm100_kernels_B64_N192_ncu.md)
# DRAM bytes of one whole step under ncu, summed over the operator's kernels (profiles/local_attention_knn_B32_N4096_ncu.md)
STEP_DRAM_BYTES = {"local": 2_108_000_000, "knn": 13_700_000, "radius": None}


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


def dist_setup(gpus: int):
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


def max_over_ranks(x: float, world: int, dev) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x: float, world: int, dev) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


# --------------------------------------------------------------------------------------------
# the reference arm / CPU baseline: oracle port of the reference's torch path on the host cores
# --------------------------------------------------------------------------------------------
def cpu_simplicial(sample_molecules: int, steps: int, warmup: int, seed: int = 0) -> dict:
    """Times the oracle (torch restatement of the reference's dense path, fp32, all host threads) on the
    first ``sample_molecules`` molecules of the benchmark batch."""
    from matterformer_b200 import synthetic
    from oracle.simplicial_ref import SimplicialInputs, simplicial_forward_backward

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    t = synthetic.config2(seed=seed)
    sel = slice(0, sample_molecules)
    inp = SimplicialInputs(**{n: t[n][sel].float() for n in NAMES}, query_valid=t["valid"][sel],
                           pair_key_valid=t["valid"][sel])  # fmt: skip
    go = t["grad_out"][sel].float()
    flops = synthetic.simplicial_flops(t["num_atoms"][sel], 8, 64)["total"]
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        simplicial_forward_backward(inp, go)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    return {"value": flops / sec / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"first {sample_molecules} of the 64 molecules (atoms {t['num_atoms'][sel].tolist()}), fp32, "
                      f"oracle port of the reference torch path, {len(times)} timed passes, {sec:.2f} s per pass",
            "ms_per_step": sec * 1e3}  # fmt: skip


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 3))
    warm = max(1, min(args.warmup, 1))
    res = cpu_simplicial(sample_molecules=4, steps=steps, warmup=warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "simplicial_fwd_bwd_B64_N192_H8_D64 (bounded sample)", "l2": "cpu"},
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def run_simplicial(args, world, rank, local) -> dict:
    import matterformer_b200 as mfb
    from matterformer_b200 import _lib, synthetic

    dev = torch.device(f"cuda:{local}")
    # replicas: the kernel workloads do not shard, every rank runs the same seeded batch (one replica per GPU)
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
    evs = []
    for _ in range(args.steps):
        flush.zero_()  # L2 flush between timed steps (outside the timed events)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        evs.append((e0, e1))
    barrier(world)
    clocks = sampler.stop()
    _lib.profile_enable(False)
    dev_ms = sum(a.elapsed_time(b) for a, b in evs)
    fwd_ms, fwd_n = _lib.profile_read(0)
    bwd_ms, bwd_n = _lib.profile_read(1)
    total_ms = max_over_ranks(dev_ms, world, dev)
    total_flops = sum_over_ranks(fl["total"], world, dev)
    value = total_flops * args.steps / (total_ms * 1e-3) / 1e12

    # ---- end to end through the public API with host buffers (pinned), copies inside the timed region
    host_in = [t[n].pin_memory() for n in NAMES] + [t["grad_out"].pin_memory()]
    host_out = [torch.empty_like(t["q"]).pin_memory() for _ in range(6)]
    h2d = sum(h.numel() * h.element_size() for h in host_in)
    d2h = sum(h.numel() * h.element_size() for h in host_out)

    # three streams (host-to-device, kernels, device-to-host) and two sets of device buffers: the copies of
    # neighbouring steps overlap the kernels; every step still moves all of its inputs and outputs
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

    peaks = measured_peaks()
    bwd_tflops = fl["bwd"] * bwd_n / (bwd_ms * 1e-3) / 1e12 if bwd_ms > 0 else None
    fwd_tflops = fl["fwd"] * fwd_n / (fwd_ms * 1e-3) / 1e12 if fwd_ms > 0 else None
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"simplicial_fwd_bwd_B{args.batch}_N192_H8_D64", "atoms": "uniform[20,181]",
                   "batch_per_gpu": args.batch, "multi_gpu": "replicas: the same seeded batch on every rank",
                   "l2": "flushed between timed steps (512 MiB write)", "flops": "valid atoms only, 14*D*H*sum n^3",
                   "pct_of_measured_bf16_peak": 100.0 * value / world / peaks["tflops"]},
        "roofline": {"bound": "tensor", "achieved": bwd_tflops, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": (bwd_tflops / peaks["tflops"]) if bwd_tflops else None, "traffic": BWD_KERNEL_DRAM_BYTES,
                     "kernel": "simplicial_bwd_sm100_kernel", "peak_source": peaks["source"] + " (burst)",
                     "kernel_ms": bwd_ms / max(bwd_n, 1), "fwd_kernel_tflops": fwd_tflops,
                     "fwd_kernel_ms": fwd_ms / max(fwd_n, 1)},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": 8 * args.steps,  # forward: extent, order, main; backward: extent, order, delta, main, finalize
        "clocks": clocks,
    }  # fmt: skip
    return line


def run_sparse(args, world, rank, local) -> dict:
    """HBM-bound workloads: radius block-sparse attention (fwd+bwd), local-window attention (fwd+bwd), kNN."""
    import matterformer_b200 as mfb
    from matterformer_b200 import synthetic

    dev = torch.device(f"cuda:{local}")
    peaks = measured_peaks()
    flush = torch.empty(L2_FLUSH_BYTES, device=dev, dtype=torch.uint8)
    launches = 0
    if args.workload == "knn":
        t = synthetic.config4(seed=0, with_qkv=False)
        pos, cell, na = t["pos"].to(dev), mfb.lattice_latent_to_cell(t["lattice"]).to(dev), t["num_atoms"].to(dev)
        step = lambda: mfb.knn_topk(pos, cell, na, k=16)  # noqa: E731
        units = pos.shape[0] * pos.shape[1]
        bytes_alg = units * (12 + 16 * 4 + 16 * 4)
        metric, unit, name, launches = "periodic kNN k=16 points/s", "points/s", "knn_B32_N4096_k16", 7  # grid, zero, count, scan, fill, search, padded rows
    else:
        if args.workload == "radius":
            t = synthetic.config3(seed=0)
            blocks = mfb.build_radius_blocks(t["pos"].to(dev), t["lattice"].to(dev), t["num_atoms"].to(dev), t["cutoff"])
            q, k, v = (t[n].to(dev).requires_grad_(True) for n in ("q", "k", "v"))
            fwd = lambda: mfb.radius_block_sparse_attention(q, k, v, blocks)  # noqa: E731
            name = "radius_attn_fwd_bwd_B16_N1024_H8_D64_cutoff6"
        else:
            t = synthetic.config4(seed=0)
            q, k, v = (t[n].to(dev).requires_grad_(True) for n in ("q", "k_", "v"))
            na = t["num_atoms"].to(dev)
            fwd = lambda: mfb.local_window_attention(q, k, v, na, window=64)  # noqa: E731
            name = "local_attn_fwd_bwd_B32_N4096_H8_D64_w64"
        go = t["grad_out"].to(dev)

        def step():
            out = fwd()
            return torch.autograd.grad(out, [q, k, v], go)

        units = q.shape[0] * q.shape[2]
        nbytes = q.numel() * 2
        bytes_alg = 4 * nbytes + 8 * nbytes  # fwd: q,k,v,o; bwd: q,k,v,o,do + dq,dk,dv
        metric, unit, launches = f"{args.workload} attention fwd+bwd atoms/s", "atoms/s", 3  # forward, dq (+ delta), dk+dv
    for _ in range(args.warmup):
        flush.zero_()
        step()
    barrier(world)
    sampler = ClockSampler(local)
    sampler.start()
    evs = []
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        evs.append((e0, e1))
    barrier(world)
    clocks = sampler.stop()
    ms = max_over_ranks(sum(a.elapsed_time(b) for a, b in evs), world, dev)
    value = units * world * args.steps / (ms * 1e-3)
    gbs = bytes_alg * args.steps / (ms * 1e-3) / 1e9
    return {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if args.workload == "knn" else "bf16", "data": "synthetic",
        "config": {"workload": name, "l2": "flushed between timed steps (512 MiB write)"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "traffic": STEP_DRAM_BYTES[args.workload], "peak_source": peaks["source"],
                     "note": "whole step (all kernels of the op) over algorithmic bytes"},
        "gpu_launches": launches * args.steps, "clocks": clocks,
    }  # fmt: skip


def trunk_flops_per_step(num_atoms: torch.Tensor, d: int = 512, layers: int = 12) -> float:
    """Model FLOPs of one EDM step (forward + backward = 3x forward) on valid tokens only: linear layers
    n*312*d^2, six simplicial cores 4*n^3*d each, six MHA cores 4*n^2*d each, adaLN 12*12*d^2 per molecule."""
    n = num_atoms.double()
    fwd = (n * 312 * d * d + (layers // 2) * 4 * n**3 * d + (layers // 2) * 4 * n**2 * d + 12 * layers * d * d).sum()
    return 3.0 * float(fwd)


def run_trunk(args, world, rank, local) -> dict:
    """Dense-token trunk, EDM denoising step forward + backward + AdamW, data parallel: global batch 1024 split
    evenly over the ranks (strong scaling), NCCL all-reduce of the gradients overlapped with backward."""
    from matterformer_b200 import synthetic
    from matterformer_b200.dp import build_edm_net, edm_train_step, shard_batch, wrap_data_parallel
    from matterformer_b200.trunk import EDMLoss

    dev = torch.device(f"cuda:{local}")
    global_batch = args.batch if args.batch != 64 else 1024
    full = synthetic.config5_batch(global_batch, seed=0)
    num_atoms = full.pop("num_atoms")
    host = {k: v.pin_memory() for k, v in shard_batch(full, rank, world).items()}
    batch = {k: v.to(dev) for k, v in host.items()}
    net = build_edm_net(seed=0).to(dev)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):  # DDP built on the stream the step will be captured on
        ddp = wrap_data_parallel(net, dev)
    torch.cuda.current_stream().wait_stream(side)
    opt = torch.optim.AdamW(net.parameters(), lr=1e-4, fused=True, capturable=not args.no_graph)
    loss_fn = EDMLoss(sigma_data=1.0)
    torch.manual_seed(1234 + rank)
    mode = "eager"
    step = lambda b=None: edm_train_step(ddp, loss_fn, opt, batch if b is None else b)  # noqa: E731
    if not args.no_graph:
        from matterformer_b200.dp import GraphedTrainStep

        graphed = GraphedTrainStep(ddp, loss_fn, opt, batch, warmup=max(11, args.warmup))
        step, mode = graphed, "cuda_graph"
    for _ in range(args.warmup):
        step()
    barrier(world)
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier(world)
    clocks = sampler.stop()
    ms = max_over_ranks(e0.elapsed_time(e1), world, dev)
    value = global_batch * args.steps / (ms * 1e-3)
    # end to end: the shard comes from pinned host memory every step and the loss is read back
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    e0.record()
    for _ in range(args.steps):
        if mode == "cuda_graph":
            float(step(host))
        else:
            float(step({k: v.to(dev, non_blocking=True) for k, v in host.items()}))
    e1.record()
    barrier(world)
    e2e_ms = max_over_ranks(e0.elapsed_time(e1), world, dev)
    peaks = measured_peaks()
    tf = trunk_flops_per_step(num_atoms) * args.steps / (ms * 1e-3) / 1e12
    params = sum(p.numel() for p in net.parameters())
    return {
        "metric": "trunk EDM step molecules/s", "value": value, "unit": "molecules/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "trunk_edm_step_L12_d512_H8_alternating_mha_simplicial", "global_batch": global_batch,
                   "atoms": "uniform[9,29]", "params": params, "parallelism": f"dp{world}", "launch": mode,
                   "l2": "working set (weights + optimizer state + activations) exceeds L2"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["tflops"] * world, "unit": "TFLOP/s",
                     "frac": tf / (peaks["tflops"] * world), "traffic": None, "peak_source": peaks["source"],
                     "note": "whole step, model FLOPs on valid tokens / step time / (n_gpus * bf16 peak)"},
        "e2e": {"value": global_batch * args.steps / (e2e_ms * 1e-3), "unit": "molecules/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": 6 * (2 + 4) * args.steps, "clocks": clocks,
    }  # fmt: skip


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="simplicial", choices=["simplicial", "radius", "local", "knn", "trunk"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="trunk workload: launch the step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--batch", type=int, default=64, help="molecules per GPU (simplicial workload; 64 = the benchmark)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the package has no CPU fallback)")
    world, rank, local = dist_setup(args.gpus)
    if args.workload == "simplicial":
        line = run_simplicial(args, world, rank, local)
    elif args.workload == "trunk":
        line = run_trunk(args, world, rank, local)
    else:
        line = run_sparse(args, world, rank, local)
    if rank == 0:
        if world == 1 and args.workload == "simplicial" and not args.no_cpu_baseline:
            res = cpu_simplicial(sample_molecules=4, steps=2, warmup=1)
            line["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
