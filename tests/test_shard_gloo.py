"""Host-side logic of the column-sharded path with two CPU ranks over gloo:
each rank computes its slice (with the oracle standing in for the device
kernel), the slices are all-gathered and interleaved exactly as the plugin's
qmatmul_sharded does, and the result equals the unsharded one bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest

from mlx_b200.shard import ShardSpec, gather_layout, shard_rows

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_spec():
    s = ShardSpec(11008, 8)
    assert s.n_local == 1376 and s.rows(0) == (0, 1376) and s.rows(7) == (9632, 11008)
    with pytest.raises(ValueError):
        ShardSpec(11008, 3)
    with pytest.raises(ValueError):
        s.rows(8)
    a = np.arange(24).reshape(8, 3)
    assert np.array_equal(np.concatenate([shard_rows(a, r, 4) for r in range(4)]), a)
    st = np.arange(2 * 3 * 4).reshape(2, 3, 4)
    y = gather_layout(st, 2, 3, 4)
    assert y.shape == (3, 8) and np.array_equal(y[1, 4:], st[1, 1])


def _worker(rank, world, port, out):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, N, bits, group = 3, 256, 64, 4, 64
        wq, s, b = O.make_layer(N, K, bits, group, O.BF16, config_id=21)
        x = O.make_x(M, K, O.BF16, config_id=21)
        y_local = O.qmatmul_ref(x, shard_rows(wq, rank, world), shard_rows(s, rank, world),
                                shard_rows(b, rank, world), bits, group)
        t = torch.from_numpy(y_local.view(np.uint8).copy())  # raw bytes, as the plugin gathers them
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        staging = torch.stack(parts).numpy().view(np.uint16).reshape(world, M, N // world)
        y = gather_layout(staging, world, M, N // world)
        full = O.qmatmul_ref(x, wq, s, b, bits, group)
        out.put((rank, bool(np.array_equal(y, full))))
    finally:
        dist.destroy_process_group()


def test_two_rank_all_gather_matches_unsharded():
    import torch.multiprocessing as mp
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == {0: True, 1: True}
