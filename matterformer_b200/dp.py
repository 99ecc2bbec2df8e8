"""Data-parallel training step for the trunk: one process per GPU, gradients all-reduced over NCCL.

The reference has no distributed code (its launch scripts request one GPU); molecules are independent
units, so the global batch is split evenly across ranks, every rank runs the full model and the only
exchange per step is the gradient all-reduce, bucketed and overlapped with backward by
``torch.nn.parallel.DistributedDataParallel``.  The step itself follows the reference's loop
(scripts/train_qm9_edm.py:592-613): autocast forward of the EDM loss, backward, gradient clipping, AdamW.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
from torch import nn

from .trunk import EDMLoss, EDMModel, EDMPreconditioner


def shard_batch(batch: dict, rank: int, world: int) -> dict:
    """Contiguous, equal shard of every (B, ...) tensor of ``batch`` for ``rank``; B must divide by ``world``."""
    b = next(iter(batch.values())).shape[0]
    if b % world:
        raise ValueError(f"global batch {b} does not divide by world size {world}")
    per = b // world
    return {k: v[rank * per : (rank + 1) * per] for k, v in batch.items()}


def wrap_data_parallel(net: nn.Module, device: Optional[torch.device] = None, bucket_mb: int = 25) -> nn.Module:
    """DDP when a process group with more than one rank exists, else the module itself."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return net
    ids = [device.index] if device is not None and device.type == "cuda" else None
    return nn.parallel.DistributedDataParallel(net, device_ids=ids, bucket_cap_mb=bucket_mb, gradient_as_bucket_view=True)


def build_edm_net(*, d_model: int = 512, n_heads: int = 8, n_layers: int = 12, simplicial_impl: str = "auto",
                  simplicial_precision: str = "bf16_tc", sigma_data: float = 1.0, seed: int = 0) -> EDMPreconditioner:  # fmt: skip
    """The trunk workload's network: 12 layers alternating MHA / 2-simplicial attention, random init."""
    torch.manual_seed(seed)
    model = EDMModel(d_model=d_model, n_heads=n_heads, n_layers=n_layers, simplicial_impl=simplicial_impl,
                     simplicial_precision=simplicial_precision)  # fmt: skip
    return EDMPreconditioner(model, sigma_data=sigma_data)


def edm_train_step(net: nn.Module, loss_fn: EDMLoss, optimizer: torch.optim.Optimizer, batch: dict, *,
                   autocast_dtype: Optional[torch.dtype] = torch.bfloat16, clip: float = 1.0, **loss_kwargs):  # fmt: skip
    """One optimisation step on this rank's shard; returns the detached loss."""
    device_type = batch["coords"].device.type
    optimizer.zero_grad(set_to_none=True)
    with torch.autocast(device_type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
        loss, _ = loss_fn(net, batch["atom_types"], batch["coords"], batch["pad_mask"], **loss_kwargs)
    loss.backward()
    if clip:
        torch.nn.utils.clip_grad_norm_(net.parameters(), clip)
    optimizer.step()
    return loss.detach()


class GraphedTrainStep:
    """One EDM training step captured in a CUDA graph and replayed.

    The trunk step is hundreds of small kernels; at a per-GPU batch of 128 molecules the host cannot launch them
    as fast as the GPU retires them, so the step is recorded once (forward, backward with the gradient
    all-reduce, clipping, AdamW) and replayed.  Inputs live in static buffers that :meth:`__call__` refreshes.
    Needs an optimizer built with ``capturable=True``; with more than one rank the DDP wrapper must have run at
    least 11 eager steps on the capture stream first (PyTorch's requirement for capturing NCCL collectives).
    """

    def __init__(self, net: nn.Module, loss_fn: EDMLoss, optimizer: torch.optim.Optimizer, example: dict, *,
                 autocast_dtype: Optional[torch.dtype] = torch.bfloat16, clip: float = 1.0, warmup: int = 11) -> None:  # fmt: skip
        self.static = {k: v.clone() for k, v in example.items()}
        self.stream = torch.cuda.Stream()
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            for _ in range(max(warmup, 3)):
                edm_train_step(net, loss_fn, optimizer, self.static, autocast_dtype=autocast_dtype, clip=clip)
        torch.cuda.current_stream().wait_stream(self.stream)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=self.stream):
            self.loss = edm_train_step(net, loss_fn, optimizer, self.static, autocast_dtype=autocast_dtype, clip=clip)

    def __call__(self, batch: Optional[dict] = None) -> torch.Tensor:
        if batch is not None:
            for k, v in batch.items():
                self.static[k].copy_(v, non_blocking=True)
        self.graph.replay()
        return self.loss
