"""Host-side logic of the column-sharded path with two CPU ranks over gloo:
each rank computes its slice (with the oracle standing in for the device
kernel), the slices are all-gathered and interleaved exactly as the plugin's
qmatmul_sharded does, and the result equals the unsharded one bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest

from mlx_b200.shard import ShardSpec, batch_layout, gather_layout, place_columns, readback_share, shard_rows

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


def test_batch_layout_and_readback_shares():
    offs, total = batch_layout([1, 4, 8, 16, 3], 11008 * 8)
    assert offs[0] == 0 and all(o % 16 == 0 for o in offs) and total == (1 + 4 + 8 + 16 + 3) * 11008 * 8 * 2
    assert all(offs[i + 1] - offs[i] == M * 11008 * 8 * 2 for i, M in enumerate([1, 4, 8, 16]))
    offs, total = batch_layout([1, 2], 20, itemsize=2)          # 40-byte rows: padded up to the alignment
    assert offs == [0, 48] and total == 48 + 80
    for world in (1, 2, 3, 8):
        for total in (4096, 1000003, 255):
            spans = [readback_share(r, world, total) for r in range(world)]
            assert spans[0][0] == 0 and sum(n for _, n in spans) == total
            assert all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert all(o % 256 == 0 for o, _ in spans)
    with pytest.raises(ValueError):
        readback_share(2, 2, 100)


def _batch_worker(rank, world, port, out):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        K, N, bits, group, Ms = 256, 64, 4, 64, [1, 3, 8, 2]
        nl = N // world
        offs, total = batch_layout(Ms, N)
        mine = np.zeros(total, np.uint8)      # this rank's copy of the result buffer
        want = np.zeros(total, np.uint8)
        for i, M in enumerate(Ms):
            wq, s, b = O.make_layer(N, K, bits, group, O.BF16, config_id=22, layer=i)
            x = O.make_x(M, K, O.BF16, config_id=22, tag=i)
            y_local = O.qmatmul_ref(x, shard_rows(wq, rank, world), shard_rows(s, rank, world), shard_rows(b, rank, world), bits, group)
            # every rank's columns of this item reach every rank (here: gathered; on the GPUs: stored by the kernels)
            t = torch.from_numpy(y_local.view(np.uint8).copy())
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t)
            for r in range(world):
                place_columns(mine, offs[i], parts[r].numpy().view(np.uint16).reshape(M, nl), r, world)
            want[offs[i]:offs[i] + M * N * 2] = O.qmatmul_ref(x, wq, s, b, bits, group).view(np.uint8).reshape(-1)
        # the hosts read the results back once between them: every rank its share; put together they are the whole
        off, n = readback_share(rank, world, total, align=16)
        share = torch.zeros(total, dtype=torch.uint8)
        share[off:off + n] = torch.from_numpy(mine[off:off + n].copy())
        dist.all_reduce(share)               # (disjoint shares: the sum is their union)
        out.put((rank, bool(np.array_equal(mine, want)), bool(np.array_equal(share.numpy(), want))))
    finally:
        dist.destroy_process_group()


def test_two_rank_batched_outputs_and_shares():
    import torch.multiprocessing as mp
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_batch_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert res == [(0, True, True), (1, True, True)]
