"""Batches of variable-size molecules under padded-size and attention-cost budgets.

Same behaviour and constructor as the reference's ``GeomDrugsPaddedBatchSampler``
(src/matterformer/data/geom_drugs.py:113-212): molecules are ordered by atom count (globally when not shuffling, inside
shuffled buckets otherwise), then cut greedily into batches so that no batch exceeds ``max_examples_per_batch`` molecules,
``max_padded_atoms_per_batch`` = max_atoms x batch padded atoms, or ``max_attention_cost_per_batch`` = max_atoms^2 x batch.
With the same ``random`` seed it yields the same batches as the reference.

One budget is added: ``max_tile_steps_per_batch`` bounds the work the row-packed tensor-core simplicial kernels really do
for the batch -- the sum over its molecules of (query ranges x steps x key slabs) from ``mf_simplicial_row_plan`` -- which,
unlike max_atoms^2 x batch, does not charge for padding the kernels skip.
"""
from __future__ import annotations

import random
from typing import Iterator, Optional, Sequence

import torch


def simplicial_tile_steps(num_atoms: int) -> int:
    """Tile-steps of the backward kernel for one molecule and one head (the forward needs at most as many)."""
    from . import _lib

    if num_atoms <= 0:
        return 0
    tiles, _, _, steps = _lib.simplicial_row_plan(min(num_atoms, 192), min(num_atoms, 192))
    return tiles * steps * ((min(num_atoms, 192) + 127) // 128)


class AttentionCostBatchSampler(torch.utils.data.Sampler):
    def __init__(self, num_atoms: Sequence[int] | torch.Tensor, *, max_examples_per_batch: int,
                 max_padded_atoms_per_batch: Optional[int] = None, max_attention_cost_per_batch: Optional[int] = None,
                 max_tile_steps_per_batch: Optional[int] = None, shuffle: bool = True, drop_last: bool = False,
                 bucket_size_multiplier: int = 32) -> None:  # fmt: skip
        super().__init__()
        counts = torch.as_tensor(num_atoms, dtype=torch.long)
        if counts.numel() == 0:
            raise ValueError("num_atoms must not be empty")
        if max_examples_per_batch <= 0:
            raise ValueError("max_examples_per_batch must be positive")
        for name, cap in (("max_padded_atoms_per_batch", max_padded_atoms_per_batch),
                          ("max_attention_cost_per_batch", max_attention_cost_per_batch),
                          ("max_tile_steps_per_batch", max_tile_steps_per_batch)):  # fmt: skip
            if cap is not None and cap <= 0:
                raise ValueError(f"{name} must be positive when set")
        if max_padded_atoms_per_batch is None and max_attention_cost_per_batch is None and max_tile_steps_per_batch is None:
            raise ValueError("At least one batch budget must be set")
        self.num_atoms = counts
        self._counts = counts.tolist()
        self.max_examples_per_batch = int(max_examples_per_batch)
        self.max_padded_atoms_per_batch = max_padded_atoms_per_batch
        self.max_attention_cost_per_batch = max_attention_cost_per_batch
        self.max_tile_steps_per_batch = max_tile_steps_per_batch
        self.shuffle = bool(shuffle)
        self.drop_last = bool(drop_last)
        self.bucket_size = max(self.max_examples_per_batch * int(bucket_size_multiplier), self.max_examples_per_batch)
        self._steps = [simplicial_tile_steps(n) for n in self._counts] if max_tile_steps_per_batch is not None else None
        self._length: Optional[int] = None

    def _by_size(self, indices: list[int]) -> list[int]:
        return sorted(indices, key=lambda i: (self._counts[i], i))

    def _order(self) -> list[int]:
        indices = list(range(len(self._counts)))
        if not self.shuffle:
            return self._by_size(indices)
        random.shuffle(indices)
        out: list[int] = []
        for lo in range(0, len(indices), self.bucket_size):
            out.extend(self._by_size(indices[lo : lo + self.bucket_size]))
        return out

    def _cut(self, order: list[int]) -> list[list[int]]:
        batches: list[list[int]] = []
        batch: list[int] = []
        widest, steps = 0, 0
        for i in order:
            n = self._counts[i]
            new_widest, size = max(widest, n), len(batch) + 1
            new_steps = steps + (self._steps[i] if self._steps is not None else 0)
            over = size > self.max_examples_per_batch
            over |= self.max_padded_atoms_per_batch is not None and new_widest * size > self.max_padded_atoms_per_batch
            over |= self.max_attention_cost_per_batch is not None and new_widest * new_widest * size > self.max_attention_cost_per_batch
            over |= self.max_tile_steps_per_batch is not None and new_steps > self.max_tile_steps_per_batch
            if batch and over:
                if not self.drop_last or len(batch) == self.max_examples_per_batch:
                    batches.append(batch)
                batch, widest, steps = [i], n, (self._steps[i] if self._steps is not None else 0)
            else:
                batch.append(i)
                widest, steps = new_widest, new_steps
        if batch and not self.drop_last:
            batches.append(batch)
        return batches

    def __iter__(self) -> Iterator[list[int]]:
        batches = self._cut(self._order())
        if self.shuffle:
            random.shuffle(batches)
        yield from batches

    def __len__(self) -> int:
        if self._length is None:
            self._length = len(self._cut(self._by_size(list(range(len(self._counts))))))
        return self._length
