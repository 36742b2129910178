"""Helper of test_gpu_symm.py (not collected by pytest): run under torchrun with one rank per GPU.

Every rank keeps a column slice of a few layers, runs the decode matmul that delivers its columns to all ranks
(qmatmul_sharded_push, then several per call with qmatmul_sharded_push_batch), and rank 0 compares the gathered result with the unsharded matmul, bit for bit.  The
shapes include few rows of W with a long K, where the decode kernel splits K over CTAs and the tiles are
finished -- and sent to the peers -- by whichever CTA arrives last.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mlx_b200  # noqa: E402
import oracle as O  # noqa: E402
from mlx_b200 import BF16  # noqa: E402
from mlx_b200.plugin import SymmBuffer  # noqa: E402
from mlx_b200.shard import batch_layout  # noqa: E402

SHAPES = [  # (M, K, N_local, bits, group)
    (8, 11008, 512, 4, 64),    # split-K
    (16, 8192, 48, 4, 32),     # split-K, 16 rows of x
    (1, 4096, 1024, 4, 64),
    (5, 2048, 2752, 8, 128),
    (16, 4096, 11008, 4, 64),
    (300, 2048, 384, 8, 32),   # prefill GEMM: tiles stored into every rank's copy from the epilogue
    (64, 1024, 144, 4, 64),
]

BATCHES = [  # (K, N_local, bits, group, [M of every item])
    (4096, 1376, 4, 64, [1, 4, 8, 16, 3, 16, 8, 1, 12, 5]),
    (11008, 512, 4, 64, [8, 2, 16]),   # split-K: single pushes at the items' offsets
    (2048, 2752, 8, 128, [7, 9, 16, 1]),
]
PROLOGUES = [  # (M, K, N_local, bits, group, prologue): 1 = rms-norm, 2 = sum of three column blocks
    (8, 4096, 1536, 4, 64, 1),
    (8, 4096, 512, 4, 64, 2),
    (3, 2048, 2752, 8, 128, 1),
    (5, 8192, 256, 4, 64, 2),   # sum3 with K split over CTAs
]


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    plugin = mlx_b200.Plugin(require_gpu=True)
    ctx = plugin.context(local)
    for case, (M, K, nl, bits, group) in enumerate(SHAPES):
        N = nl * world
        wq, s, b = O.make_layer(N, K, bits, group, O.BF16, config_id=8, layer=case)
        x = O.make_x(M, K, O.BF16, config_id=8, tag=case)
        sl = slice(rank * nl, (rank + 1) * nl)
        bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq[sl]), ctx.upload(s[sl]), ctx.upload(b[sl])
        sb = SymmBuffer(ctx, rank, world, (M, N), np.uint16)
        mine = torch.tensor(list(sb.export()), dtype=torch.uint8, device="cuda")
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        sb.attach([bytes(t.cpu().tolist()) for t in every])
        dist.barrier()
        for rep in range(20):  # the same buffer again and again: the inbox hand-shake is part of the test
            sb.qmatmul(bx, bw, bs, bb, M, K, nl, bits, group, BF16)
        ctx.sync()
        got = sb.to_host()
        dist.barrier()
        if rank == 0:
            fw, fs, fb = ctx.upload(wq), ctx.upload(s), ctx.upload(b)
            ref = ctx.empty((M, N), np.uint16)
            ctx.qmatmul(bx, fw, fs, fb, ref, M, K, N, bits, group, BF16, BF16, BF16)
            want = ref.to_host()
            if not np.array_equal(got, want):
                bad = np.argwhere(got != want)
                print(f"MISMATCH case {case} {(M, K, nl, bits, group)}: {len(bad)} elements, first {bad[:4].tolist()}", flush=True)
                os._exit(3)
            for h in (fw, fs, fb, ref):
                h.free()
        dist.barrier()
        sb.free()
        for h in (bx, bw, bs, bb):
            h.free()
    # Several matmuls per call (qmatmul_sharded_push_batch): the outputs one after another in one buffer, the call
    # repeated into the same buffer; the second shape is one whose K the decode kernel splits over CTAs, which
    # runs as single pushes at the items' offsets inside the call.
    for case, (K, nl, bits, group, Ms) in enumerate(BATCHES):
        N = nl * world
        layers = [O.make_layer(N, K, bits, group, O.BF16, config_id=9, layer=10 * case + i) for i in range(len(Ms))]
        xs = [O.make_x(M, K, O.BF16, config_id=9, tag=10 * case + i) for i, M in enumerate(Ms)]
        sl = slice(rank * nl, (rank + 1) * nl)
        up = [(ctx.upload(x), ctx.upload(l[0][sl]), ctx.upload(l[1][sl]), ctx.upload(l[2][sl])) for x, l in zip(xs, layers)]
        offs, total = batch_layout(Ms, N)
        sb = SymmBuffer(ctx, rank, world, (total // 2,), np.uint16)
        mine = torch.tensor(list(sb.export()), dtype=torch.uint8, device="cuda")
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        sb.attach([bytes(t.cpu().tolist()) for t in every])
        dist.barrier()
        for rep in range(10):
            sb.qmatmul_batch([u[0] for u in up], [u[1] for u in up], [u[2] for u in up], [u[3] for u in up], offs, Ms,
                             K, nl, bits, group, BF16)
        ctx.sync()
        got = [sb.item_to_host(offs[i], (M, N), np.uint16) for i, M in enumerate(Ms)]
        dist.barrier()
        if rank == 0:
            for i, M in enumerate(Ms):
                fw, fs, fb = ctx.upload(layers[i][0]), ctx.upload(layers[i][1]), ctx.upload(layers[i][2])
                ref = ctx.empty((M, N), np.uint16)
                ctx.qmatmul(up[i][0], fw, fs, fb, ref, M, K, N, bits, group, BF16, BF16, BF16)
                if not np.array_equal(got[i], ref.to_host()):
                    bad = np.argwhere(got[i] != ref.to_host())
                    print(f"MISMATCH batch {case} item {i} (M={M}): {len(bad)} elements, first {bad[:4].tolist()}", flush=True)
                    os._exit(3)
                for h in (fw, fs, fb, ref):
                    h.free()
        dist.barrier()
        sb.free()
        for u in up:
            for h in u:
                h.free()
    # Prologues on a sharded layer (qmatmul_sharded_push_pro): x is a wider buffer (three column blocks for sum3);
    # the gathered result must be the unsharded qmatmul_pro's, bit for bit (the row statistics of the rms-norm are
    # computed by every CTA from the same fragments in the same order, whatever its share of the columns).
    from mlx_b200.plugin import PRO_RMS_NORM, PRO_SUM3
    for case, (M, K, nl, bits, group, which) in enumerate(PROLOGUES):
        N = nl * world
        x_ld = 3 * K if which == PRO_SUM3 else K + 64
        wq, s, b = O.make_layer(N, K, bits, group, O.BF16, config_id=10, layer=case)
        x = O.make_x(M, x_ld, O.BF16, config_id=10, tag=case)
        sl = slice(rank * nl, (rank + 1) * nl)
        bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq[sl]), ctx.upload(s[sl]), ctx.upload(b[sl])
        sb = SymmBuffer(ctx, rank, world, (M, N), np.uint16)
        mine = torch.tensor(list(sb.export()), dtype=torch.uint8, device="cuda")
        every = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        sb.attach([bytes(t.cpu().tolist()) for t in every])
        dist.barrier()
        for rep in range(5):
            sb.qmatmul_pro(bx, bw, bs, bb, M, K, nl, bits, group, BF16, which, x_ld, 1e-6)
        ctx.sync()
        got = sb.to_host()
        dist.barrier()
        if rank == 0:
            fw, fs, fb = ctx.upload(wq), ctx.upload(s), ctx.upload(b)
            ref = ctx.empty((M, N), np.uint16)
            ctx.qmatmul_pro(bx, fw, fs, fb, ref, M, K, N, bits, group, BF16, which, x_ld, 1e-6)
            if not np.array_equal(got, ref.to_host()):
                bad = np.argwhere(got != ref.to_host())
                print(f"MISMATCH prologue case {case}: {len(bad)} elements, first {bad[:4].tolist()}", flush=True)
                os._exit(3)
            for h in (fw, fs, fb, ref):
                h.free()
        dist.barrier()
        sb.free()
        for h in (bx, bw, bs, bb):
            h.free()
    # The batched call again with the ranks drifting apart: no barrier between the calls, two alternating sets of
    # activations (so that a store that came late or early would show), and EVERY rank checks the whole buffer
    # after EVERY call against the unsharded matmuls it has computed itself.
    import time
    K, nl, bits, group = 4096, 1376, 4, 64
    N = nl * world
    Ms = [1, 8, 4, 16, 3, 16, 8, 1, 12, 5, 2, 7]
    layers = [O.make_layer(N, K, bits, group, O.BF16, config_id=11, layer=i) for i in range(len(Ms))]
    sl = slice(rank * nl, (rank + 1) * nl)
    loc = [(ctx.upload(l[0][sl]), ctx.upload(l[1][sl]), ctx.upload(l[2][sl])) for l in layers]
    xsets = [[ctx.upload(O.make_x(M, K, O.BF16, config_id=11, tag=10 * v + i)) for i, M in enumerate(Ms)] for v in range(2)]
    offs, total = batch_layout(Ms, N)
    want = []
    for v in range(2):
        flat = np.zeros(total // 2, np.uint16)
        for i, M in enumerate(Ms):
            fw, fs, fb = ctx.upload(layers[i][0]), ctx.upload(layers[i][1]), ctx.upload(layers[i][2])
            y = ctx.empty((M, N), np.uint16)
            ctx.qmatmul(xsets[v][i], fw, fs, fb, y, M, K, N, bits, group, BF16, BF16, BF16)
            flat[offs[i] // 2: offs[i] // 2 + M * N] = y.to_host().reshape(-1)
            for h in (fw, fs, fb, y):
                h.free()
        want.append(flat)
    sb = SymmBuffer(ctx, rank, world, (total // 2,), np.uint16)
    mine = torch.tensor(list(sb.export()), dtype=torch.uint8, device="cuda")
    every = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    sb.attach([bytes(t.cpu().tolist()) for t in every])
    dist.barrier()
    rng = np.random.default_rng(rank)
    bad = 0
    for it in range(60):
        v = it & 1
        sb.qmatmul_batch(xsets[v], [l[0] for l in loc], [l[1] for l in loc], [l[2] for l in loc], offs, Ms, K, nl, bits, group, BF16)
        if it % 3 == rank % 3:
            time.sleep(float(rng.uniform(0, 0.002)))
        if not np.array_equal(sb.to_host(), want[v]):  # (synchronises this rank only)
            bad += 1
    t = torch.tensor([bad], dtype=torch.int64, device="cuda")
    dist.all_reduce(t)
    ctx.sync()
    dist.barrier()
    if int(t.item()):
        if rank == 0:
            print(f"MISMATCH drifting ranks: {int(t.item())} calls left a buffer that differs", flush=True)
        os._exit(3)
    sb.free()
    if rank == 0:
        print(f"SYMM_RANKS_OK world={world} cases={len(SHAPES)} batches={len(BATCHES)} prologues={len(PROLOGUES)} drifting_calls=60", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
