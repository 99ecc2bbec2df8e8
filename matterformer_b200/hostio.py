"""Forward + backward of the 2-simplicial attention kernels for callers whose tensors live in host memory.

A step copies q, k1, v1, k2, v2 and grad_out from pinned host buffers to the GPU, runs the forward
and backward kernels and copies out and the five gradients back.  Run back to back on one stream the
three parts take about as long as each other; :class:`HostPipelinedSimplicial` puts them on three
streams (host-to-device, compute, device-to-host) with two sets of device buffers, so that the copies
of neighbouring steps overlap the kernels of the current one and the step time approaches the longest
of the three parts.  Every step still moves all of its inputs and outputs.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .simplicial import cuda_simplicial_attention_backward, cuda_simplicial_attention_forward


class HostPipelinedSimplicial:
    """``submit(host_inputs, host_outputs)`` enqueues one step; ``finish()`` waits for all of them.

    ``host_inputs`` = (q, k1, v1, k2, v2, grad_out) pinned host tensors of shape (B,H,N,D);
    ``host_outputs`` = (out, dq, dk1, dv1, dk2, dv2) pinned host tensors that receive the results.
    Masks stay on the device.  ``depth`` steps may be in flight at once.
    """

    def __init__(self, device: torch.device, *, query_valid: torch.Tensor, pair_key_valid: torch.Tensor,
                 pair_valid: Optional[torch.Tensor] = None, precision: str = "bf16_tc", depth: int = 2) -> None:  # fmt: skip
        self.device = torch.device(device)
        self.masks = dict(query_valid=query_valid, pair_key_valid=pair_key_valid, pair_valid=pair_valid)
        self.precision = precision
        self.depth = max(1, int(depth))
        self.s_in = torch.cuda.Stream(self.device)
        self.s_compute = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self._slots = [dict(inputs=None, results=None, ev_in=torch.cuda.Event(), ev_compute=torch.cuda.Event(),
                            ev_out=torch.cuda.Event(), used=False) for _ in range(self.depth)]  # fmt: skip
        self._next = 0

    def submit(self, host_inputs: Sequence[torch.Tensor], host_outputs: Sequence[torch.Tensor]) -> None:
        slot = self._slots[self._next]
        self._next = (self._next + 1) % self.depth
        if slot["inputs"] is None:
            with torch.cuda.stream(self.s_in):
                slot["inputs"] = [torch.empty(h.shape, dtype=h.dtype, device=self.device) for h in host_inputs]
        # host -> device: the slot's buffers are free once the kernels of its previous step have run
        with torch.cuda.stream(self.s_in):
            if slot["used"]:
                self.s_in.wait_event(slot["ev_compute"])
            for d, h in zip(slot["inputs"], host_inputs):
                d.copy_(h, non_blocking=True)
            slot["ev_in"].record(self.s_in)
        # kernels: the previous results of this slot must have left for the host before they are released
        with torch.cuda.stream(self.s_compute):
            self.s_compute.wait_event(slot["ev_in"])
            if slot["used"]:
                self.s_compute.wait_event(slot["ev_out"])
            q, k1, v1, k2, v2, grad_out = slot["inputs"]
            out, lse, out32 = cuda_simplicial_attention_forward(q, k1, v1, k2, v2, precision=self.precision,
                                                                **self.masks)  # fmt: skip
            grads = cuda_simplicial_attention_backward(grad_out, q, k1, v1, k2, v2, out32, lse,
                                                       precision=self.precision, **self.masks)  # fmt: skip
            slot["results"] = (out, *grads[:5])
            slot["ev_compute"].record(self.s_compute)
        # device -> host
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(slot["ev_compute"])
            for h, g in zip(host_outputs, slot["results"]):
                h.copy_(g, non_blocking=True)
            slot["ev_out"].record(self.s_out)
        slot["used"] = True

    def finish(self) -> None:
        self.s_out.synchronize()
        self.s_compute.synchronize()
        self.s_in.synchronize()
