"""Batches of independent structures over several GPUs (one process per GPU): data-parallel, no collective.

Each rank evaluates a contiguous range of the graphs, chosen so that the ranks hold about the same number of atoms;
nothing is exchanged in the energy+force path (replaces the batching of so3lr/base_calculator.py:57-122 and
so3lr/cli/so3lr_eval.py for more than one device).  `gather_results` collects per-graph numbers on every rank for reporting.
"""
from __future__ import annotations

import numpy as np


def shard_graphs(graph_start, world: int, rank: int):
    """(first, last) graph indices [first, last) of `rank`: contiguous ranges with balanced atom counts.
    `graph_start` holds the first atom of every graph plus the total atom count (n_graphs + 1 entries)."""
    gs = np.asarray(graph_start, dtype=np.int64)
    n_graphs, n_atoms = len(gs) - 1, int(gs[-1])
    # boundary k goes to the graph whose start is nearest to k/world of the atoms
    cuts = [int(np.searchsorted(gs, round(k * n_atoms / world), side="left")) for k in range(world + 1)]
    cuts[0], cuts[-1] = 0, n_graphs
    for k in range(1, world + 1):
        cuts[k] = max(cuts[k], cuts[k - 1])
    return cuts[rank], cuts[rank + 1]


class ShardedBatch:
    """The graphs of one rank.  `atomic_numbers`, `positions` and `graph_start` describe the whole batch (identical on
    every rank); only the local slice is sent to the device."""

    def __init__(self, atomic_numbers, graph_start, world: int, rank: int, *, lr_cutoff=1000.0, damping=2.0, device=0, system_factory=None):
        gs = np.asarray(graph_start, dtype=np.int64)
        self.first, self.last = shard_graphs(gs, world, rank)
        self.a0, self.a1 = int(gs[self.first]), int(gs[self.last])
        self.local_start = (gs[self.first:self.last + 1] - self.a0).astype(np.int32)
        self.n_graphs_local = self.last - self.first
        self.system = None
        if self.n_graphs_local > 0:
            Z = np.asarray(atomic_numbers, dtype=np.int32)[self.a0:self.a1]
            if system_factory is None:
                from .engine import System
                system_factory = System
            self.system = system_factory(Z, None, cutoff_lr=lr_cutoff, damping=damping, lr_format="sparse",
                                         graph_start=self.local_start if self.n_graphs_local > 1 else None, device=device)

    def compute_host(self, positions):
        """Energy (per local graph), forces (local atoms), charges, Hirshfeld ratios, dipoles of this rank's graphs."""
        if self.system is None:
            return dict(energy=np.zeros(0), forces=np.zeros((0, 3), np.float32), partial_charges=np.zeros(0, np.float32),
                        hirshfeld_ratios=np.zeros(0, np.float32), dipole_vec=np.zeros((0, 3), np.float32))
        return self.system.compute_host(np.asarray(positions, dtype=np.float32)[self.a0:self.a1])


def gather_results(local: dict, world: int):
    """Concatenate the per-rank result dictionaries in rank order on every rank (reporting only; uses
    torch.distributed.all_gather_object, so it works with gloo and nccl process groups alike)."""
    if world == 1:
        return local
    import torch.distributed as dist
    parts = [None] * world
    dist.all_gather_object(parts, local)
    return {k: np.concatenate([p[k] for p in parts]) for k in local}
