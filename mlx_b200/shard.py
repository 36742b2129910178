"""Column sharding of a quantized layer over the GPUs of one box.

Rank r of ``world`` owns output columns [r*Nl, (r+1)*Nl): the matching rows
of Wq / scales / biases never move; x is replicated; the output slices are
all-gathered.  Pure host bookkeeping (no GPU needed to test it).
"""
from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class ShardSpec:
    N: int
    world: int

    def __post_init__(self):
        if self.world < 1 or self.N % self.world:
            raise ValueError(f"N={self.N} is not divisible by world={self.world}")

    @property
    def n_local(self):
        return self.N // self.world

    def rows(self, rank):
        if not 0 <= rank < self.world:
            raise ValueError(f"rank {rank} outside [0,{self.world})")
        return rank * self.n_local, (rank + 1) * self.n_local


def shard_rows(a, rank, world):
    """Rows of a per-output-row array (Wq, scales, biases) owned by ``rank``."""
    lo, hi = ShardSpec(a.shape[0], world).rows(rank)
    return np.ascontiguousarray(a[lo:hi])


def gather_layout(staging, world, M, n_local):
    """The column interleave that follows the all-gather:
    staging[r][m][j] -> y[m][r*n_local + j]."""
    s = np.asarray(staging).reshape(world, M, n_local)
    return np.ascontiguousarray(np.transpose(s, (1, 0, 2)).reshape(M, world * n_local))
