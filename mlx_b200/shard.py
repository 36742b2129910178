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


def batch_layout(Ms, n_total, itemsize=2, align=16):
    """Byte offsets of the outputs y_i[M_i, n_total] of a batched sharded call inside one symmetric buffer, one
    after another (each a multiple of ``align``, as qmatmul_sharded_push_batch wants), and the bytes in all."""
    offsets, total = [], 0
    for M in Ms:
        if M < 1:
            raise ValueError("every item needs at least one row of x")
        offsets.append(total)
        total += -(-(M * n_total * itemsize) // align) * align
    return offsets, total


def readback_share(rank, world, total, align=256):
    """[offset, offset + length) of the result buffer that ``rank`` copies back to its host when the ranks read
    the results back once between them: equal aligned parts, the last rank takes the remainder."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside [0,{world})")
    part = (total // world) // align * align
    off = rank * part
    return off, (part if rank < world - 1 else total - off)


def place_columns(buf, offset, y_local, rank, world, itemsize=2):
    """What a rank's batched kernel does to every rank's copy of the buffer for one item: its columns
    [rank*Nl, (rank+1)*Nl) of y[M, world*Nl] at byte ``offset`` (a host model of the peer stores)."""
    M, nl = y_local.shape
    view = buf[offset:offset + M * nl * world * itemsize].view(y_local.dtype).reshape(M, nl * world)
    view[:, rank * nl:(rank + 1) * nl] = y_local
