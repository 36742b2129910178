"""Symmetric buffers and the decode matmul that does its own all-gather (symm_*, qmatmul_sharded_push).

With one GPU only world = 1 can run as a kernel: ranks that wait for one another must not share a GPU.
The multi-rank path is checked (bit for bit, every rank's columns) by bench.py on 2, 4 and 8 GPUs, and
this file runs that check itself when the box has at least two GPUs.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

from mlx_b200 import BF16, BackendError
from mlx_b200 import plugin as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_world_of_one_equals_plain_qmatmul(ctx, oracle):
    M, K, N = 8, 1024, 256
    wq, s, b = oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=8, layer=3)
    x = oracle.make_x(M, K, oracle.BF16, config_id=8, tag=3)
    bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    y = ctx.empty((M, N), np.uint16)
    ctx.qmatmul(bx, bw, bs, bb, y, M, K, N, 4, 64, BF16, BF16, BF16)
    sb = P.SymmBuffer(ctx, 0, 1, (M, N), np.uint16)
    assert len(sb.export()) == P.SYMM_HANDLE_BYTES
    sb.qmatmul(bx, bw, bs, bb, M, K, N, 4, 64, BF16)
    assert np.array_equal(sb.to_host(), y.to_host())
    with pytest.raises(BackendError):  # N_local must be whole 16-column tiles
        sb.qmatmul(bx, bw, bs, bb, M, K, N - 8, 4, 64, BF16)
    sb.free()
    for h in (bx, bw, bs, bb, y):
        h.free()


def test_world_of_one_batch_equals_plain_qmatmul(ctx, oracle):
    """qmatmul_sharded_push_batch with a world of one rank: every item's output, at its offset of the buffer, is
    the plain qmatmul's; overlapping or misplaced outputs are refused."""
    K, N = 2048, 512
    Ms = [1, 8, 16, 3, 12]
    layers = [oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=8, layer=i) for i in range(len(Ms))]
    xs = [oracle.make_x(M, K, oracle.BF16, config_id=8, tag=i) for i, M in enumerate(Ms)]
    up = [(ctx.upload(x), ctx.upload(l[0]), ctx.upload(l[1]), ctx.upload(l[2])) for x, l in zip(xs, layers)]
    offs, total = [], 0
    for M in Ms:
        offs.append(total)
        total += M * N * 2
    sb = P.SymmBuffer(ctx, 0, 1, (total // 2,), np.uint16)
    sb.qmatmul_batch([u[0] for u in up], [u[1] for u in up], [u[2] for u in up], [u[3] for u in up], offs, Ms, K, N, 4, 64, BF16)
    for i, M in enumerate(Ms):
        y = ctx.empty((M, N), np.uint16)
        ctx.qmatmul(*up[i], y, M, K, N, 4, 64, BF16, BF16, BF16)
        assert np.array_equal(sb.item_to_host(offs[i], (M, N), np.uint16), y.to_host()), i
        y.free()
    args = ([u[0] for u in up[:2]], [u[1] for u in up[:2]], [u[2] for u in up[:2]], [u[3] for u in up[:2]])
    with pytest.raises(BackendError):  # the second output starts inside the first
        sb.qmatmul_batch(*args, [0, 16], Ms[:2], K, N, 4, 64, BF16)
    with pytest.raises(BackendError):  # not a multiple of 16 bytes
        sb.qmatmul_batch(*args, [0, 8 + N * 2], Ms[:2], K, N, 4, 64, BF16)
    with pytest.raises(BackendError):  # past the end of the buffer
        sb.qmatmul_batch(*args, [0, total - 32], Ms[:2], K, N, 4, 64, BF16)
    sb.free()
    for u in up:
        for h in u:
            h.free()


def test_attach_is_required_and_checks_rank_order(ctx):
    sb = P.SymmBuffer(ctx, 0, 2, (4, 64), np.uint16)
    dummy = ctx.empty((4, 64), np.uint16)
    with pytest.raises(BackendError):
        sb.qmatmul(dummy, dummy, dummy, dummy, 4, 64, 32, 4, 64, BF16)  # not attached
    h = sb.export()
    with pytest.raises(BackendError):
        sb.attach([h, h])  # second handle says rank 0, not 1
    sb.free()
    dummy.free()


def test_two_ranks_bit_exact(plugin):
    if plugin.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "1", "--warmup", "3", "--reps", "2",
           "--kernel-only"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    assert '"verified": "all ranks' in r.stdout


def test_ranks_bit_exact_including_split_k(plugin):
    """Several shapes (among them few rows of W with a long K, which the decode kernel splits over CTAs) pushed
    twenty times each into the same buffer by every rank: tests/symm_ranks_check.py compares on rank 0."""
    n = plugin.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    n = 2 if n < 4 else 4
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr", "127.0.0.1",
           "--master-port", "29537", os.path.join(ROOT, "tests", "symm_ranks_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0 and "SYMM_RANKS_OK" in r.stdout, (r.stdout[-1500:], r.stderr[-1500:])


WAIT_RUNS_OUT = r"""
import sys
sys.path.insert(0, %r)
import numpy as np
import mlx_b200
from mlx_b200 import BF16, BackendError
from mlx_b200 import plugin as P
import oracle as O
plugin = mlx_b200.Plugin(require_gpu=True)
ctx = plugin.context(0)
M, K, Nl, batch = %d, 1024, 128, %d
wq, s, b = O.make_layer(Nl, K, 4, 64, O.BF16, config_id=8)
x = O.make_x(M, K, O.BF16, config_id=8)
bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b)
# rank 0 of a world of two; "rank 1" is a second buffer on the same GPU on which nothing is ever launched
rows = 2 * M if batch else M
mine, other = P.SymmBuffer(ctx, 0, 2, (rows, 2 * Nl), np.uint16), P.SymmBuffer(ctx, 1, 2, (rows, 2 * Nl), np.uint16)
hs = [mine.export(), other.export()]
mine.attach(hs)
other.attach(hs)
before = mine.to_host().copy()
if batch:                                                   # (returns: the wait happens on the device)
    mine.qmatmul_batch([bx, bx], [bw, bw], [bs, bs], [bb, bb], [0, M * 2 * Nl * 2], [M, M], K, Nl, 4, 64, BF16)
else:
    mine.qmatmul(bx, bw, bs, bb, M, K, Nl, 4, 64, BF16)
try:
    ctx.sync()
    print("NO_ERROR")
except BackendError as e:
    print("SYNC_ERROR", e)
after = mine.to_host()
print("PEER_COLUMNS_UNTOUCHED", bool(np.array_equal(after[:, Nl:], before[:, Nl:])))
ctx.sync()                                                  # the context stays usable
y = ctx.empty((M, Nl), np.uint16)
ctx.qmatmul(bx, bw, bs, bb, y, M, K, Nl, 4, 64, BF16, BF16, BF16)
err, _ = O.rel_err(y.to_host(), O.qmatmul_truth(x, wq, s, b, 4, 64))
print("STILL_WORKS", bool(err <= 1e-2))
"""


@pytest.mark.parametrize("M,batch", [(8, 0), (64, 0), (8, 1)])
def test_a_wait_for_a_peer_runs_out_and_is_reported(M, batch):
    """Bounded device-side waits, exercised the harmless way: the 'peer' is a buffer nobody launches on, the limit
    is 50 ms (LUXCUDA_PEER_WAIT_MS).  The kernel gives up by itself, the next sync reports INTERNAL, nothing faults
    or hangs, and the context keeps working.  M = 8: the decode kernel's wait for the peer's ready word; M = 64: the
    rank barrier around the prefill GEMM; batch: the batched decode kernel's wait for the ready word (it then sends
    nothing and reports).  In a process of its own: having given up once, a process stops waiting
    for peers."""
    env = dict(os.environ, LUXCUDA_PEER_WAIT_MS="50")
    r = subprocess.run([sys.executable, "-c", WAIT_RUNS_OUT % (ROOT, M, batch)], capture_output=True, text=True, timeout=120, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "SYNC_ERROR" in r.stdout and "NO_ERROR" not in r.stdout, r.stdout
    assert "STILL_WORKS True" in r.stdout, r.stdout
    if M <= 16:
        assert "PEER_COLUMNS_UNTOUCHED True" in r.stdout, r.stdout
