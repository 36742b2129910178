"""Prefill-regime GEMM (tcgen05 + TMEM) against the oracle, through the C ABI.
Same bars as the decode tests: outputs within 1e-2 (bf16 compute) of the
fp64-accumulated truth over the same bf16 dequantised weights."""
import numpy as np
import pytest

from mlx_b200 import BF16, F32
from test_gpu_parity import check, run_qmatmul

pytestmark = pytest.mark.gpu

SHAPES = [
    # M, K, N, bits, group
    (32, 64, 128, 4, 64),        # one tile, one k-stage
    (32, 256, 128, 4, 64),       # one tile, exactly the pipeline depth
    (17, 320, 128, 4, 64),       # M tail inside the x tile (rows 17..31 are zero fill)
    (48, 512, 200, 4, 64),       # N tail (rows clamped, stores masked), bm = 48
    (128, 1024, 256, 4, 32),     # group 32: two groups per k-stage
    (130, 768, 384, 4, 128),     # group 128
    (300, 1024, 384, 4, 64),     # two x tiles of 160 rows
    (64, 256, 128, 8, 128),      # 8-bit
    (96, 1024, 300, 8, 64),
    (256, 2048, 1024, 8, 32),
    (512, 4096, 2048, 4, 64),    # many tiles per CTA: stage wrap-around
]


@pytest.mark.parametrize("M,K,N,bits,group", SHAPES)
def test_prefill_bf16(ctx, oracle, M, K, N, bits, group):
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=3, layer=K, proj=N)
    x = oracle.make_x(M, K, oracle.BF16, config_id=3, layer=K, tag=M)
    for y_dtype in (BF16, F32):
        y, kern = run_qmatmul(ctx, x, wq, s, b, bits, group, y_dtype)
        assert kern.startswith("qmm_tc"), kern
        t = oracle.qmatmul_truth(x, wq, s, b, bits, group)
        err, nerr = oracle.rel_err(y, t)
        assert err <= oracle.TOL[oracle.BF16], (err, nerr)
        if y_dtype == F32:
            assert nerr <= 1e-5  # fp32 accumulation in TMEM: far inside the bf16 bar before output rounding


def test_prefill_matches_decode_kernel(ctx, oracle):
    """The GEMM and the GEMV use the same dequantised weights: rows of a big-M
    result agree with the decode kernel on the same rows to fp32 summation order."""
    M, K, N = 64, 1024, 512
    wq, s, b = oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=3)
    x = oracle.make_x(M, K, oracle.BF16, config_id=3)
    yg, kern = run_qmatmul(ctx, x, wq, s, b, 4, 64, F32)
    assert kern.startswith("qmm_tc")
    yv, kern = run_qmatmul(ctx, x[:8], wq, s, b, 4, 64, F32)
    assert kern.startswith("qmv_mma")
    assert np.abs(yg[:8] - yv).max() <= 1e-5 * np.abs(yv).max()


def test_prefill_full_size_sampled(ctx, oracle):
    """Benchmark shape (M=2048, K=4096, N=4096): one-hot rows of x pick out
    dequantised weight columns exactly; random rows are checked against the
    oracle on a sample of rows."""
    M, K, N = 2048, 4096, 4096
    wq, s, b = oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=3)
    x = oracle.make_x(M, K, oracle.BF16, config_id=3)
    hot = {5: 0, 700: 63, 1300: 2049, 2047: 4095}
    for m, k in hot.items():
        x[m] = 0
        x[m, k] = 0x3F80
    y, kern = run_qmatmul(ctx, x, wq, s, b, 4, 64, BF16)
    assert kern.startswith("qmm_tc")
    w = oracle.dequantize(wq, s, b, K, 4, 64, oracle.BF16)
    for m, k in hot.items():
        assert np.array_equal(y[m], w[:, k])
    rows = [0, 1, 255, 256, 1023, 1500, 2046]
    t = oracle.qmatmul_truth(x[rows], wq, s, b, 4, 64)
    err, _ = oracle.rel_err(y[rows], t)
    assert err <= oracle.TOL[oracle.BF16], err


def test_large_8bit_full_size_sampled(ctx, oracle):
    """The 8-bit large-GEMM configuration on one GPU (M=512, K=8192, N=28672, group 128): one-hot rows of x
    pick out dequantised weight columns exactly; random rows are checked against the oracle on a sample of
    output columns (the oracle is run on the matching rows of W only)."""
    M, K, N, bits, group = 512, 8192, 28672, 8, 128
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=4)  # 8-bit default scale range: U(1e-4, 2e-3)
    x = oracle.make_x(M, K, oracle.BF16, config_id=4)
    hot = {3: 0, 200: 127, 317: 4097, 511: 8191}
    for m, k in hot.items():
        x[m] = 0
        x[m, k] = 0x3F80
    y, kern = run_qmatmul(ctx, x, wq, s, b, bits, group, BF16)
    assert kern.startswith("qmm_tc"), kern
    cols = np.r_[0:128, 3584 - 64:3584 + 64, 14336 - 64:14336 + 64, 20000:20128, N - 128:N]
    w = oracle.dequantize(wq[cols], s[cols], b[cols], K, bits, group, oracle.BF16)
    for m, k in hot.items():
        assert np.array_equal(y[m, cols], w[:, k])
    rows = [0, 1, 127, 128, 255, 256, 400, 510]
    t = oracle.qmatmul_truth(x[rows], wq[cols], s[cols], b[cols], bits, group)
    err, _ = oracle.rel_err(y[np.ix_(rows, cols)], t)
    assert err <= oracle.TOL[oracle.BF16], err


@pytest.mark.parametrize("M,K,N,bits,group", [(256, 2048, 1024, 8, 32), (256, 2048, 1024, 4, 64), (130, 1024, 300, 8, 128)])
def test_prefill_is_repeatable(ctx, oracle, M, K, N, bits, group):
    """The kernel hands tiles between warps, the copy engine and the tensor core through barriers only: the same
    launch repeated many times must give the same bits every time (a missed hand-over shows up here long
    before it shows up in a tolerance check)."""
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=3, layer=K, proj=N)
    x = oracle.make_x(M, K, oracle.BF16, config_id=3, layer=K, tag=M)
    bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    ys = [ctx.empty((M, N), np.uint16) for _ in range(4)]
    ctx.qmatmul(bx, bw, bs, bb, ys[0], M, K, N, bits, group, BF16, BF16, BF16)
    first = ys[0].to_host()
    check(oracle, first, x, wq, s, b, bits, group, oracle.BF16)
    bad = 0
    for rep in range(60):
        for y in ys:
            ctx.qmatmul(bx, bw, bs, bb, y, M, K, N, bits, group, BF16, BF16, BF16)
        for y in ys:
            bad += not np.array_equal(y.to_host(), first)
    for h in (bx, bw, bs, bb, *ys):
        h.free()
    assert bad == 0, f"{bad} of 240 launches differed from the first"


@pytest.mark.parametrize("schedule", ["streamk", "tiles", "pairs"])
@pytest.mark.parametrize("M,K,N,bits,group", [(64, 4096, 4096, 4, 64), (512, 4096, 2048, 4, 64), (300, 1024, 384, 4, 64),
                                                  (512, 8192, 3584, 8, 128), (32, 64, 128, 4, 64), (2048, 1024, 4096, 4, 64)])
def test_both_schedules(ctx, oracle, monkeypatch, schedule, M, K, N, bits, group):
    """The launch either gives every CTA whole tiles, or gives pairs of CTAs (one MMA stream for two SMs) pairs of
    tiles, or splits the sequence of (tile, k-stage) units evenly over the CTAs, partial accumulators of a split tile
    being added in a fixed order by the CTA that starts the tile.  The host picks one per shape; here each is forced
    in turn: all meet the bar, and all are repeatable bit for bit (the flags of the partial-accumulator exchange are
    left reset by every launch)."""
    monkeypatch.setenv("LUXCUDA_QMM_SCHEDULE", "streamk" if schedule == "streamk" else "tiles")
    monkeypatch.setenv("LUXCUDA_QMM_PAIR", "1" if schedule == "pairs" else "0")
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=3, layer=K, proj=N)
    x = oracle.make_x(M, K, oracle.BF16, config_id=3, layer=K, tag=M)
    bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    y = ctx.empty((M, N), np.uint16)
    ctx.qmatmul(bx, bw, bs, bb, y, M, K, N, bits, group, BF16, BF16, BF16)
    assert ctx.last_kernel().startswith("qmm_tc") and (schedule == "tiles") == ctx.last_kernel().endswith(("<4>", "<8>"))
    first = y.to_host()
    rows = np.unique(np.r_[0:min(M, 4), M // 2, M - 1])
    cols = np.unique(np.r_[0:min(N, 64), N // 2:N // 2 + 32, N - 64:N])
    t = oracle.qmatmul_truth(x[rows], wq[cols], s[cols], b[cols], bits, group)
    err, _ = oracle.rel_err(first[np.ix_(rows, cols)], t)
    assert err <= oracle.TOL[oracle.BF16], err
    for _ in range(20):
        ctx.qmatmul(bx, bw, bs, bb, y, M, K, N, bits, group, BF16, BF16, BF16)
        assert np.array_equal(y.to_host(), first)
    for h in (bx, bw, bs, bb, y):
        h.free()
