"""Row-block sharding of one matrix over the GPUs of a node, x replicated.

Rank p owns the contiguous rows [bounds[p], bounds[p+1]) (nnz-balanced, asp_partition_rows_by_nnz),
builds its own format on that block with global column indices and runs the single-GPU path. A
single SpMV needs no communication. In repeated-SpMV mode (x <- A x) every iteration ends with an
all-gather of the ranks' y slices into the next x: the slices differ in length, so they are gathered
into a buffer of `world * max_rows` elements and compacted with one copy per rank. Kernels only ever
read local memory; NCCL moves remote data into it first.

The reference is single-GPU (code_builder.cc:1483-1489); this module has no counterpart there.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


class ShardedSpmv:
    """`local_spmv(x, y_local)` computes this rank's slice: x is the full replicated vector
    (torch tensor, length n_cols), y_local a tensor of at least bounds[rank+1]-bounds[rank] elements.
    On a GPU it is `PlanGroup.spmv` on the tensors' pointers; the CPU tests pass a host function."""

    def __init__(self, local_spmv, bounds, rank: int, world: int, dtype, device, group=None):
        self.local_spmv = local_spmv
        self.bounds = [int(b) for b in bounds]
        self.rank, self.world, self.group = rank, world, group
        self.rows = [self.bounds[p + 1] - self.bounds[p] for p in range(world)]
        self.max_rows = max(self.rows)
        self.n = self.bounds[-1]
        self.y_local = torch.zeros(self.max_rows, dtype=dtype, device=device)
        self.gathered = torch.zeros(world * self.max_rows, dtype=dtype, device=device) if world > 1 else None

    def spmv_slice(self, x: torch.Tensor) -> torch.Tensor:
        """y[bounds[rank]:bounds[rank+1]] for the replicated x (no communication)."""
        self.local_spmv(x, self.y_local)
        return self.y_local[: self.rows[self.rank]]

    def gather_into(self, x_next: torch.Tensor) -> None:
        """All ranks' current y slices -> x_next (full length), in row order."""
        if self.world == 1:
            x_next[: self.rows[0]].copy_(self.y_local[: self.rows[0]])
            return
        dist.all_gather_into_tensor(self.gathered, self.y_local, group=self.group)
        for p in range(self.world):
            x_next[self.bounds[p] : self.bounds[p + 1]].copy_(self.gathered[p * self.max_rows : p * self.max_rows + self.rows[p]])

    def iterate(self, x0: torch.Tensor, iters: int, scratch: torch.Tensor | None = None) -> torch.Tensor:
        """x <- A x, `iters` times (square matrices); returns the final replicated x."""
        a = x0
        b = scratch if scratch is not None else torch.empty_like(x0)
        for _ in range(iters):
            self.local_spmv(a, self.y_local)
            self.gather_into(b)
            a, b = b, a
        return a


def balanced_bounds_from_degrees(deg: np.ndarray, parts: int) -> np.ndarray:
    """Row bounds with about sum(deg) / parts non-zeros per part, from per-row counts."""
    from .graph import partition_rows_by_nnz

    indptr = np.zeros(deg.shape[0] + 1, dtype=np.int64)
    np.cumsum(deg, out=indptr[1:])
    return partition_rows_by_nnz(indptr, parts)
