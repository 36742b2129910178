"""Quantized-linear chain (decode regime, M = 8): consecutive matmuls where each output is the next
input, rms-norm between layers -- the shape of configuration 5, reduced to a few layers.

Consecutive decode launches of a context are chained as programmatic dependent launches (the next kernel
fetches weights while the previous one drains and waits before it reads x), so the chain is also the
test of that dependency: back-to-back launches must equal, bit for bit, the same launches with a full
synchronisation between them, and each step must match the oracle on the input the step actually saw.
"""
import numpy as np
import pytest

from mlx_b200 import BF16
from mlx_b200 import plugin as P

pytestmark = pytest.mark.gpu

D, FF, M = 1024, 2816, 8          # model width, MLP width (11008/4), rows of x
PROJ = [("q", D, D), ("o", D, D), ("gate", FF, D), ("down", D, FF)]   # (name, N, K), applied in sequence


def _layers(ctx, oracle, n_layers):
    out = []
    for layer in range(n_layers):
        for pi, (_, N, K) in enumerate(PROJ):
            wq, s, b = oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=5, layer=layer, proj=pi)
            out.append((N, K, wq, s, b, ctx.upload(wq), ctx.upload(s), ctx.upload(b)))
    return out


def _run(ctx, layers, x0, sync_every_call):
    """Returns the list of (input, output) arrays of every matmul, as the device saw them."""
    bufs = {D: [ctx.empty((M, D), np.uint16) for _ in range(2)], FF: [ctx.empty((M, FF), np.uint16)]}
    norm = ctx.empty((M, D), np.uint16)
    cur = ctx.upload(x0)
    trace, flip = [], 0
    per_layer = len(PROJ)
    for i, (N, K, _, _, _, bw, bs, bb) in enumerate(layers):
        if i % per_layer == 0:  # renormalise the residual stream at the start of each layer
            ctx.rms_norm(cur, norm, M, D, 1e-6, BF16, BF16)
            src = norm
        else:
            src = cur
        dst = bufs[N][flip % len(bufs[N])]
        flip += 1
        if dst is src:
            dst = bufs[N][flip % len(bufs[N])]
            flip += 1
        ctx.qmatmul(src, bw, bs, bb, dst, M, K, N, 4, 64, BF16, BF16, BF16)
        assert ctx.last_kernel().startswith("qmv_mma")
        if sync_every_call:
            ctx.sync()
            trace.append((src.to_host((M, K), np.uint16), dst.to_host((M, N), np.uint16)))
        else:
            trace.append((src, dst, (M, K), (M, N)))
        cur = dst
    ctx.sync()
    final = cur.to_host((M, layers[-1][0]), np.uint16)
    for b in bufs[D] + bufs[FF] + [norm]:
        b.free()
    return trace, final


def test_chain_matches_oracle_step_by_step(ctx, oracle):
    layers = _layers(ctx, oracle, 2)
    x0 = oracle.make_x(M, D, oracle.BF16, config_id=5)
    trace, _ = _run(ctx, layers, x0, sync_every_call=True)
    for (N, K, wq, s, b, *_), (xin, yout) in zip(layers, trace):
        t = oracle.qmatmul_truth(xin, wq, s, b, 4, 64)
        err, nerr = oracle.rel_err(yout, t)
        assert err <= oracle.TOL[oracle.BF16], (N, K, err, nerr)
    for l in layers:
        for h in l[5:]:
            h.free()


def test_back_to_back_launches_equal_synchronised_launches(ctx, oracle):
    layers = _layers(ctx, oracle, 3)
    x0 = oracle.make_x(M, D, oracle.BF16, config_id=5, tag=1)
    _, ref = _run(ctx, layers, x0, sync_every_call=True)
    for _ in range(5):  # timing-dependent faults would not show on every run
        _, got = _run(ctx, layers, x0, sync_every_call=False)
        assert np.array_equal(got, ref)
    for l in layers:
        for h in l[5:]:
            h.free()


def test_weights_written_just_before_use(ctx, oracle):
    """A matmul right behind the kernel that produces its weights (quantize) must see them: such a
    launch is never chained to the decode launch before it."""
    N, K = 512, 1024
    rng = np.random.default_rng(7)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    x = oracle.make_x(M, K, oracle.BF16, config_id=5, tag=2)
    bw_f, bzero, bx = ctx.upload(w), ctx.upload(np.zeros((N, K), np.float32)), ctx.upload(x)
    y0, y1 = ctx.empty((M, N), np.uint16), ctx.empty((M, N), np.uint16)
    wq, s, b = ctx.empty((N, K // 8), np.uint32), ctx.empty((N, K // 64), np.uint16), ctx.empty((N, K // 64), np.uint16)
    bwarm = [ctx.upload(a) for a in oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=5, layer=9)]
    results = []
    for sync in (True, False):
        ctx.quantize(bzero, wq, s, b, N, K, 4, 64, BF16)  # stale weights: all zero
        ctx.sync()
        ctx.qmatmul(bx, *bwarm, y0, M, K, N, 4, 64, BF16, BF16, BF16)  # a decode launch right before
        ctx.quantize(bw_f, wq, s, b, N, K, 4, 64, BF16)
        if sync:
            ctx.sync()
        ctx.qmatmul(bx, wq, s, b, y1, M, K, N, 4, 64, BF16, BF16, BF16)
        results.append(y1.to_host())
    assert np.array_equal(results[0], results[1])
    assert np.any(results[0] != 0)
    for h in [bw_f, bzero, bx, y0, y1, wq, s, b] + bwarm:
        h.free()


@pytest.mark.parametrize("M,K,N,bits,group", [(1, 4096, 1024, 4, 64), (16, 2048, 528, 4, 32), (8, 8192, 96, 8, 128)])
def test_decode_is_repeatable(ctx, oracle, M, K, N, bits, group):
    """Back-to-back decode launches overlap (the next one fetches weights while the previous drains) and hand
    partial sums between warps and CTAs: repeated launches must give the same bits every time."""
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=6, layer=K, proj=N)
    x = oracle.make_x(M, K, oracle.BF16, config_id=6, layer=K, tag=M)
    bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    ys = [ctx.empty((M, N), np.uint16) for _ in range(8)]
    ctx.qmatmul(bx, bw, bs, bb, ys[0], M, K, N, bits, group, BF16, BF16, BF16)
    first = ys[0].to_host()
    bad = 0
    for rep in range(40):
        for y in ys:
            ctx.qmatmul(bx, bw, bs, bb, y, M, K, N, bits, group, BF16, BF16, BF16)
        for y in ys:
            bad += not np.array_equal(y.to_host(), first)
    for h in (bx, bw, bs, bb, *ys):
        h.free()
    assert bad == 0, f"{bad} of 320 launches differed from the first"
