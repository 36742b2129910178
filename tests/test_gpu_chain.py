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


def _bf16_ulps(a, b):
    """Distance in bf16 steps between two bf16 arrays of equal sign pattern (raw uint16)."""
    return np.abs(a.astype(np.int32) - b.astype(np.int32)).max()


def test_full_width_layer_dataflow(ctx, oracle):
    """The chain configuration's own dataflow on two layers at full width (4096 / 11008):
    a = bf16(q + k + v); o = Wo a; r = rms_norm(o); m = rms_norm(bf16(gate(r) * up(r))); d = Wd m; h' = rms_norm(d),
    q|k|v and gate|up as one launch each.  Every step is checked against the oracle on the input it actually saw;
    then the same launches back to back (no synchronisation, programmatic dependent launches) must give the same bits."""
    M, Dm, FFm, eps = 8, 4096, 11008, 1e-6
    shapes = [("qkv", 3 * Dm, Dm), ("o", Dm, Dm), ("gateup", 2 * FFm, Dm), ("down", Dm, FFm)]
    layers = []
    for l in range(2):
        ws = {}
        for pi, (name, N, K) in enumerate(shapes):
            wq, s, b = oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=5, layer=l, proj=pi)
            ws[name] = (wq, s, b, ctx.upload(wq), ctx.upload(s), ctx.upload(b), N, K)
        layers.append(ws)
    x0 = oracle.make_x(M, Dm, oracle.BF16, config_id=5)
    t = {n: ctx.empty((M, N), np.uint16) for n, N in (("h", Dm), ("qkv", 3 * Dm), ("a", Dm), ("o", Dm), ("r", Dm),
                                                       ("gateup", 2 * FFm), ("m", FFm), ("d", Dm))}

    def run(check):
        hb = ctx.upload(x0)

        def mm(ws, name, src, dst, src_shape):
            wq, s, b, bw, bs, bb, N, K = ws[name]
            ctx.qmatmul(src, bw, bs, bb, dst, M, K, N, 4, 64, BF16, BF16, BF16)
            if check:
                xin, y = src.to_host(src_shape, np.uint16), dst.to_host((M, N), np.uint16)
                err, nerr = oracle.rel_err(y, oracle.qmatmul_truth(xin, wq, s, b, 4, 64))
                assert err <= oracle.TOL[oracle.BF16], (name, err, nerr)

        cur = hb
        for ws in layers:
            mm(ws, "qkv", cur, t["qkv"], (M, Dm))
            ctx.sum3(t["qkv"], t["a"], M, Dm, 3 * Dm)
            if check:  # elementwise, one rounding: bit-exact
                assert np.array_equal(t["a"].to_host((M, Dm), np.uint16), oracle.sum3(t["qkv"].to_host((M, 3 * Dm), np.uint16), Dm))
            mm(ws, "o", t["a"], t["o"], (M, Dm))
            ctx.rms_norm(t["o"], t["r"], M, Dm, eps, BF16, BF16)
            if check:  # the row sum of squares is accumulated in another order: one bf16 step
                assert _bf16_ulps(t["r"].to_host((M, Dm), np.uint16), oracle.rms_norm(t["o"].to_host((M, Dm), np.uint16), eps=eps)) <= 1
            mm(ws, "gateup", t["r"], t["gateup"], (M, Dm))
            ctx.mul_rms_norm(t["gateup"], t["m"], M, FFm, 2 * FFm, eps)
            if check:
                assert _bf16_ulps(t["m"].to_host((M, FFm), np.uint16), oracle.mul_rms_norm(t["gateup"].to_host((M, 2 * FFm), np.uint16), FFm, eps=eps)) <= 1
            mm(ws, "down", t["m"], t["d"], (M, FFm))
            ctx.rms_norm(t["d"], t["h"], M, Dm, eps, BF16, BF16)
            if check:
                assert _bf16_ulps(t["h"].to_host((M, Dm), np.uint16), oracle.rms_norm(t["d"].to_host((M, Dm), np.uint16), eps=eps)) <= 1
            cur = t["h"]
        ctx.sync()
        out = t["h"].to_host((M, Dm), np.uint16)
        hb.free()
        return out

    ref = run(check=True)
    assert np.isfinite(oracle.from_bf16(ref)).all()
    for _ in range(3):
        assert np.array_equal(run(check=False), ref)
    for ws in layers:
        for v in ws.values():
            for h in v[3:6]:
                h.free()
    for b in t.values():
        b.free()


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


@pytest.mark.parametrize("M,K,N,bits,group", [(8, 4096, 512, 4, 64), (3, 2048, 96, 8, 128), (1, 1024, 1030, 4, 32)])
def test_prologues_equal_the_separate_steps(ctx, oracle, M, K, N, bits, group):
    """qmatmul_pro applies sum3 or the rms-norm to x while the decode kernel loads it.  sum3 is one rounding per
    element, so the fused launch must give the bits of sum3 followed by qmatmul; the rms-norm accumulates the row's
    sum of squares in another order than the stand-alone kernel (one bf16 step on a normalised value at most), so
    the fused launch is held to the oracle's bar on the oracle's normalised input, and to the same bar against the
    two-launch result."""
    eps = 1e-6
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=5, layer=K, proj=N)
    bw, bs, bb = ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    wide = oracle.make_x(M, 3 * K, oracle.BF16, config_id=5, layer=K, tag=M)     # q | k | v of one launch
    bwide = ctx.upload(wide)
    a, y_two, y_one = ctx.empty((M, K), np.uint16), ctx.empty((M, N), np.uint16), ctx.empty((M, N), np.uint16)
    # sum3
    ctx.sum3(bwide, a, M, K, 3 * K)
    ctx.qmatmul(a, bw, bs, bb, y_two, M, K, N, bits, group, BF16, BF16, BF16)
    ctx.qmatmul_pro(bwide, bw, bs, bb, y_one, M, K, N, bits, group, BF16, P.PRO_SUM3, 3 * K)
    assert ctx.last_kernel().endswith("sum3>")
    assert np.array_equal(y_one.to_host(), y_two.to_host())
    t = oracle.qmatmul_truth(oracle.sum3(wide, K), wq, s, b, bits, group)
    assert oracle.rel_err(y_one.to_host(), t)[0] <= oracle.TOL[oracle.BF16]
    # rms-norm of the first K columns of the wide buffer (row stride 3K), and of a plain [M][K] buffer
    x = np.ascontiguousarray(wide[:, :K])
    ctx.rms_norm(ctx.upload(x), a, M, K, eps, BF16, BF16)
    ctx.qmatmul(a, bw, bs, bb, y_two, M, K, N, bits, group, BF16, BF16, BF16)
    t = oracle.qmatmul_truth(oracle.rms_norm(x, eps=eps), wq, s, b, bits, group)
    for buf, ld in ((bwide, 3 * K), (ctx.upload(x), K)):
        ctx.qmatmul_pro(buf, bw, bs, bb, y_one, M, K, N, bits, group, BF16, P.PRO_RMS_NORM, ld, eps)
        assert ctx.last_kernel().endswith("rms>")
        got = y_one.to_host()
        assert oracle.rel_err(got, t)[0] <= oracle.TOL[oracle.BF16]
        assert oracle.rel_err(got, oracle.from_bf16(y_two.to_host()).astype(np.float64))[0] <= oracle.TOL[oracle.BF16]
    # repeated launches give the same bits
    first = y_one.to_host()
    for _ in range(10):
        ctx.qmatmul_pro(bwide, bw, bs, bb, y_one, M, K, N, bits, group, BF16, P.PRO_RMS_NORM, 3 * K, eps)
        assert np.array_equal(y_one.to_host(), first)


def test_prologue_refuses_what_it_does_not_take(ctx, oracle, plugin):
    K, N = 8192, 64
    wq, s, b = oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=5, layer=9)
    bw, bs, bb = ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    x16 = ctx.upload(oracle.make_x(16, K, oracle.BF16, config_id=5))
    y = ctx.empty((16, N), np.uint16)
    for M, pro in ((16, P.PRO_SUM3), (8, P.PRO_RMS_NORM)):   # more than 8 rows; K of 32 k-blocks (and split) for the norm
        with pytest.raises(P.BackendError) as ei:
            ctx.qmatmul_pro(x16, bw, bs, bb, y, M, K if pro == P.PRO_RMS_NORM else K // 4, N, 4, 64, BF16, pro, K, 1e-6)
        assert ei.value.code == P.ERR_NOT_SUPPORTED, plugin.last_error()
    with pytest.raises(P.BackendError) as ei:   # x_ld too short for three column blocks
        ctx.qmatmul_pro(x16, bw, bs, bb, y, 8, K // 4, N, 4, 64, BF16, P.PRO_SUM3, K // 2)
    assert ei.value.code == P.ERR_INVALID
