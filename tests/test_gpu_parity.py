"""Parity of the CUDA path with the oracle, through the C ABI, on a B200.

Bars (north_star): unpack and dequantised weights bit-exact; matmul outputs
within max relative error 1e-2 (bf16 compute) / 1e-4 (fp32 compute) of the
fp64-accumulated truth over the same dequantised weights and inputs, where
the error is  max_i |y_i - t_i| / max(|t_i|, 1e-2 * max|t|)  (oracle.rel_err).
"""
import glob
import os

import numpy as np
import pytest

from mlx_b200 import BF16, F32, BackendError
from mlx_b200 import plugin as P

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = sorted(p for p in glob.glob(os.path.join(GOLDEN, "*.npz")) if not p.endswith("kat_words.npz"))


def run_qmatmul(ctx, x, wq, s, b, bits, group, y_dtype, via_dispatch=False):
    M, K = x.shape
    N = wq.shape[0]
    xd, sd = P._np_dtype_code(x), P._np_dtype_code(s)
    bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    by = ctx.empty((M, N), np.uint16 if y_dtype == BF16 else np.float32)
    try:
        f = ctx.qmatmul_dispatch if via_dispatch else ctx.qmatmul
        f(bx, bw, bs, bb, by, M, K, N, bits, group, xd, sd, y_dtype)
        return by.to_host(), ctx.last_kernel()
    finally:
        for h in (bx, bw, bs, bb, by):
            h.free()


def check(oracle, y, x, wq, s, b, bits, group, dt):
    t = oracle.qmatmul_truth(x, wq, s, b, bits, group)
    err, nerr = oracle.rel_err(y, t)
    assert err <= oracle.TOL[dt], (err, nerr)
    return err


def test_kat_words_unpack(ctx):
    k = np.load(os.path.join(GOLDEN, "kat_words.npz"))
    for w, q, K, bits in ((k["w4"], k["q4"], 32, 4), (k["w8"], k["q8"], 8, 8)):
        bw, bo = ctx.upload(w), ctx.empty((1, K), np.uint8)
        ctx.unpack(bw, bo, 1, K, bits)
        assert np.array_equal(bo.to_host(), q)
        bw.free(); bo.free()


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[:-4] for p in CASES])
def test_golden(ctx, oracle, path):
    g = np.load(path)
    M, K, N, bits, group, dt = (int(g[k]) for k in ("M", "K", "N", "bits", "group", "dtype"))
    wq, s, b, x = g["wq"], g["scales"], g["biases"], g["x"]
    bw, bs, bb = ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    # unpack: bit-exact
    bq = ctx.empty((N, K), np.uint8)
    ctx.unpack(bw, bq, N, K, bits)
    assert np.array_equal(bq.to_host(), g["q"])
    # dequantised weights: bit-exact
    bo = ctx.empty((N, K), g["w"].dtype)
    ctx.dequantize(bw, bs, bb, bo, N, K, bits, group, P._np_dtype_code(s), dt)
    assert np.array_equal(bo.to_host(), g["w"])
    for h in (bw, bs, bb, bq, bo):
        h.free()
    # matmul: every output dtype, both call routes
    for y_dtype in (F32, BF16):
        for via in (False, True):
            y, kern = run_qmatmul(ctx, x, wq, s, b, bits, group, y_dtype, via_dispatch=via)
            err, _ = oracle.rel_err(y, g["truth"])
            # a bf16 output carries its own 2^-9 rounding whatever the compute dtype
            tol = oracle.TOL[dt] if y_dtype == F32 else oracle.TOL[oracle.BF16]
            assert err <= tol, (kern, err)
    # against what the reference CPU backend computed (fp32 sequential sum): both within tolerance of the
    # truth, so within the sum of the two of each other
    y, _ = run_qmatmul(ctx, x, wq, s, b, bits, group, F32)
    tmax = np.abs(g["truth"]).max()
    assert np.abs(y - g["y_refcore"]).max() <= 2 * oracle.TOL[dt] * tmax


SHAPES = [
    # M, K, N, bits, group  -- decode shapes, tails in N, one k-block, several k-blocks, odd row tiles
    (1, 256, 16, 4, 64), (1, 256, 1, 4, 64), (3, 512, 37, 4, 64), (8, 1024, 100, 4, 64), (9, 768, 50, 4, 128),
    (16, 2048, 333, 4, 64), (5, 256, 24, 4, 32), (16, 512, 31, 4, 32),
    (1, 128, 16, 8, 128), (4, 384, 19, 8, 64), (16, 1024, 77, 8, 128), (7, 256, 40, 8, 32),
    (2, 4096, 4096, 4, 64), (8, 11008, 512, 4, 64), (16, 4096, 1376, 4, 64), (1, 8192, 3584, 8, 128),
    (12, 4096, 11008, 4, 64),
]


@pytest.mark.parametrize("M,K,N,bits,group", SHAPES)
def test_decode_bf16(ctx, oracle, M, K, N, bits, group):
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=2, layer=K, proj=N)
    x = oracle.make_x(M, K, oracle.BF16, config_id=2, layer=K, tag=M)
    y, kern = run_qmatmul(ctx, x, wq, s, b, bits, group, BF16)
    assert kern.startswith("qmv_mma"), kern
    check(oracle, y, x, wq, s, b, bits, group, oracle.BF16)


@pytest.mark.parametrize("M", [1, 4, 8, 16])
def test_decode_sweep_shape(ctx, oracle, M):
    """The decode-sweep configuration itself (K=4096, N=11008, 4-bit, group 64) at each of its batch sizes."""
    K, N = 4096, 11008
    wq, s, b = oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=2)
    x = oracle.make_x(M, K, oracle.BF16, config_id=2, tag=M)
    y, kern = run_qmatmul(ctx, x, wq, s, b, 4, 64, BF16)
    assert kern.startswith("qmv_mma"), kern
    check(oracle, y, x, wq, s, b, 4, 64, oracle.BF16)


def test_decode_workspace_shared_between_split_shapes(ctx, oracle):
    """Two K-split shapes with different tile counts, one after the other on one context: the second must not
    read the first one's partials as arrival counters (the counters sit in a region of fixed size)."""
    for (M, K, N, bits, group) in ((8, 8192, 64, 4, 64), (1, 8192, 1120, 4, 64), (8, 16384, 1024, 4, 64), (1, 8192, 1120, 4, 64)):
        wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=2, layer=K, proj=N)
        x = oracle.make_x(M, K, oracle.BF16, config_id=2, layer=K, tag=M)
        y, kern = run_qmatmul(ctx, x, wq, s, b, bits, group, BF16)
        assert kern.startswith("qmv_mma"), kern
        check(oracle, y, x, wq, s, b, bits, group, oracle.BF16)


@pytest.mark.parametrize("M,K,N,bits,group", [(1, 4096, 4096, 4, 64), (4, 1024, 130, 4, 64), (2, 512, 64, 8, 128),
                                              (16, 256, 9, 4, 32), (1, 64, 5, 4, 64)])
def test_fp32_compute(ctx, oracle, M, K, N, bits, group):
    """The CPU-reference configuration (fp32 x, fp32 scales, biases = -8*scale + noise)."""
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.F32, config_id=1, bias_noise=1e-3)
    x = oracle.make_x(M, K, oracle.F32, config_id=1)
    y, kern = run_qmatmul(ctx, x, wq, s, b, bits, group, F32)
    assert kern.startswith("qmv_simt"), kern
    check(oracle, y, x, wq, s, b, bits, group, oracle.F32)
    # the reference-style CPU result (sequential fp32 sum) agrees to the sum of both tolerances
    yr = oracle.qmatmul_ref(x, wq, s, b, bits, group)
    assert np.abs(y - yr).max() <= 2e-4 * np.abs(yr).max()
    # bf16 scales with fp32 activations are widened, same rule
    s16, b16 = oracle.to_bf16(s), oracle.to_bf16(b)
    y2, _ = run_qmatmul(ctx, x, wq, s16, b16, bits, group, F32)
    check(oracle, y2, x, wq, s16, b16, bits, group, oracle.F32)


def test_fallback_shapes_bf16(ctx, oracle):
    """K not a multiple of the tensor-core k-blocks: the CUDA-core kernel takes over."""
    for (M, K, N, bits, group) in ((3, 192, 20, 4, 64), (2, 64, 7, 8, 64), (20, 96, 33, 4, 32)):
        wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=5)
        x = oracle.make_x(M, K, oracle.BF16, config_id=5)
        y, kern = run_qmatmul(ctx, x, wq, s, b, bits, group, BF16)
        assert kern.startswith("qmv_simt"), kern
        check(oracle, y, x, wq, s, b, bits, group, oracle.BF16)


def test_rows_of_x_are_independent(ctx, oracle):
    """M=1 result equals the matching row of the M=16 result bit for bit, and
    repeated rows of x give identical rows of y."""
    K, N = 1024, 200
    wq, s, b = oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=6)
    x = oracle.make_x(16, K, oracle.BF16, config_id=6)
    x[5] = x[2]
    y16, _ = run_qmatmul(ctx, x, wq, s, b, 4, 64, BF16)
    assert np.array_equal(y16[5], y16[2])
    for m in (0, 7, 15):
        y1, _ = run_qmatmul(ctx, x[m:m + 1], wq, s, b, 4, 64, BF16)
        assert np.array_equal(y1[0], y16[m])


def test_column_slices_equal_full_layer(ctx, oracle):
    """Sharding along N changes no dot product: the kernel on each column slice
    reproduces the full-layer output bit for bit (world = 2, 4, 8)."""
    M, K, N = 8, 4096, 2752
    wq, s, b = oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=8)
    x = oracle.make_x(M, K, oracle.BF16, config_id=8)
    full, _ = run_qmatmul(ctx, x, wq, s, b, 4, 64, BF16)
    for world in (2, 4, 8):
        nl = N // world
        parts = [run_qmatmul(ctx, x, wq[r * nl:(r + 1) * nl], s[r * nl:(r + 1) * nl], b[r * nl:(r + 1) * nl], 4, 64, BF16)[0]
                 for r in range(world)]
        assert np.array_equal(np.concatenate(parts, axis=1), full)


def test_linearity_and_extremes(ctx, oracle):
    """Size-independent properties at the benchmark's full decode size."""
    M, K, N = 4, 4096, 11008
    wq, s, b = oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=2)
    # x = 0 -> y = 0 ; x = e_k (one-hot) -> y[:, n] = w^[n, k] exactly (a single product, no rounding)
    x = np.zeros((M, K), np.uint16)
    ks = [0, 7, 63, 4095]
    for m, k in enumerate(ks):
        x[m, k] = 0x3F80  # 1.0
    y, _ = run_qmatmul(ctx, x, wq, s, b, 4, 64, BF16)
    w = oracle.dequantize(wq, s, b, K, 4, 64, oracle.BF16)
    for m, k in enumerate(ks):
        assert np.array_equal(y[m], w[:, k])
    y0, _ = run_qmatmul(ctx, np.zeros((M, K), np.uint16), wq, s, b, 4, 64, BF16)
    assert not y0.any()
    # all-zero and all-max codes
    for word in (0x00000000, 0xFFFFFFFF):
        wq2 = np.full_like(wq[:64], word)
        xr = oracle.make_x(2, K, oracle.BF16, config_id=9)
        y2, _ = run_qmatmul(ctx, xr, wq2, s[:64], b[:64], 4, 64, BF16)
        check(oracle, y2, xr, wq2, s[:64], b[:64], 4, 64, oracle.BF16)


def test_empty_and_invalid(ctx, oracle, plugin):
    wq, s, b = oracle.make_layer(16, 256, 4, 64, oracle.BF16, config_id=4)
    x = oracle.make_x(2, 256, oracle.BF16, config_id=4)
    bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    by = ctx.empty((2, 16), np.uint16)
    ctx.qmatmul(bx, bw, bs, bb, by, 0, 256, 16, 4, 64, BF16, BF16, BF16)  # M = 0: no-op
    ctx.qmatmul(bx, bw, bs, bb, by, 2, 256, 0, 4, 64, BF16, BF16, BF16)   # N = 0: no-op
    for bad in (dict(bits=3), dict(group=48), dict(K=250), dict(M=3), dict(N=17), dict(sb=F32), dict(xd=1)):
        a = dict(M=2, K=256, N=16, bits=4, group=64, xd=BF16, sb=BF16)
        a.update(bad)
        with pytest.raises(BackendError) as ei:
            ctx.qmatmul(bx, bw, bs, bb, by, a["M"], a["K"], a["N"], a["bits"], a["group"], a["xd"], a["sb"], BF16)
        assert ei.value.code in (P.ERR_INVALID, P.ERR_NOT_SUPPORTED)
    assert plugin.last_error()
    for h in (bx, bw, bs, bb, by):
        h.free()


def test_quantize_matches_oracle(ctx, oracle):
    w = oracle.gen_normal(77, (48, 512), 0.0, 0.05)
    for bits, group, sbd in ((4, 64, F32), (8, 128, BF16), (4, 32, BF16), (8, 64, F32), (4, 128, F32)):
        wq, s, b = oracle.quantize(w, bits, group, sbd)
        bi = ctx.upload(w)
        bw, bs, bb = ctx.empty(wq.shape, wq.dtype), ctx.empty(s.shape, s.dtype), ctx.empty(b.shape, b.dtype)
        ctx.quantize(bi, bw, bs, bb, 48, 512, bits, group, sbd)
        assert np.array_equal(bs.to_host(), s) and np.array_equal(bb.to_host(), b)
        assert np.array_equal(bw.to_host(), wq)
        for h in (bi, bw, bs, bb):
            h.free()


def test_rms_norm(ctx, oracle):
    x = oracle.make_x(8, 4096, oracle.BF16, config_id=10)
    bi, bo = ctx.upload(x), ctx.empty(x.shape, np.uint16)
    ctx.rms_norm(bi, bo, 8, 4096, 1e-6, BF16, BF16)
    got, want = oracle.from_bf16(bo.to_host()), oracle.from_bf16(oracle.rms_norm(x, eps=1e-6))
    assert np.abs(got - want).max() <= 2 ** -7 * np.abs(want).max()  # one bf16 ulp of the largest value
    bi.free(); bo.free()


@pytest.mark.parametrize("bits,group", [(4, 64), (8, 128), (4, 32)])
def test_scale_extremes_bit_exact(ctx, oracle, bits, group):
    """Scales outside the range of the fast in-register dequantiser (zero,
    subnormal, >= 2^-5, huge, negative) and right at its edges: dequantised
    weights stay bit-exact and the matmul stays within tolerance."""
    K, N = 512, 64
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=12)
    special = np.array([0.0, 1.0, 0.03125, 0.0311, 1e-39, -0.01, 3.0e4, 2.0 ** -126, 2.0 ** -120, -0.5, 0.0078125],
                       np.float32)
    sf = oracle.from_bf16(s)
    sf.reshape(-1)[:special.size * 3:3] = special
    s = oracle.to_bf16(sf)
    b = oracle.to_bf16(oracle.gen_normal(5, b.shape, 0.0, 0.05))
    bw, bs, bb = ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    bo = ctx.empty((N, K), np.uint16)
    ctx.dequantize(bw, bs, bb, bo, N, K, bits, group, BF16, BF16)
    assert np.array_equal(bo.to_host(), oracle.dequantize(wq, s, b, K, bits, group, oracle.BF16))
    for h in (bw, bs, bb, bo):
        h.free()
    x = oracle.make_x(3, K, oracle.BF16, config_id=12)
    y, kern = run_qmatmul(ctx, x, wq, s, b, bits, group, F32)
    assert kern.startswith("qmv_mma")
    check(oracle, y, x, wq, s, b, bits, group, oracle.BF16)


@pytest.mark.parametrize("K,N,bits,group,Ms", [(4096, 1200, 4, 64, [1, 4, 8, 16, 3, 12, 8, 1]), (2048, 528, 8, 128, [2, 16, 16, 7]),
                                                  (1024, 100, 4, 32, [5]), (8192, 64, 4, 64, [8, 1, 16]),
                                                  # more matmuls than CTAs (the CTAs' tile ranges rotate from one matmul to the
                                                  # next and wrap around), 4 bytes of scales per row and k-block
                                                  (2048, 272, 4, 128, [8, 1, 3, 5, 2, 7, 4, 6, 8, 1, 2, 3, 4, 5, 6, 7, 8, 1, 2, 3]),
                                                  (1024, 304, 8, 32, [1, 8, 4]), (2048, 2400, 8, 64, [6, 2, 16, 9, 1]),
                                                  (4096, 11008, 4, 64, [1, 8, 8, 3, 16])])
def test_batch_equals_single_calls(ctx, oracle, K, N, bits, group, Ms):
    """qmatmul_batch runs independent decode matmuls of one shape in as few persistent launches as their M allow (the
    last shape is one whose K the decode kernel splits over CTAs: the call then runs them one by one).  Either way
    every result must be the bits of a qmatmul call of its own, and within the bar of the oracle."""
    layers, xs, want = [], [], []
    for i, M in enumerate(Ms):
        wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=7, layer=i, proj=N)
        x = oracle.make_x(M, K, oracle.BF16, config_id=7, layer=i, tag=M)
        bw, bs, bb, bx = ctx.upload(wq), ctx.upload(s), ctx.upload(b), ctx.upload(x)
        y = ctx.empty((M, N), np.uint16)
        ctx.qmatmul(bx, bw, bs, bb, y, M, K, N, bits, group, BF16, BF16, BF16)
        got = y.to_host()
        check(oracle, got, x, wq, s, b, bits, group, oracle.BF16)
        layers.append((bw, bs, bb)); xs.append(bx); want.append(got)
        y.free()
    ys = [ctx.empty((M, N), np.uint16) for M in Ms]
    for rep in range(3):
        for y, M in zip(ys, Ms):
            y.from_host(np.zeros((M, N), np.uint16))
        ctx.qmatmul_batch(xs, [l[0] for l in layers], [l[1] for l in layers], [l[2] for l in layers], ys, Ms, K, N, bits, group, BF16)
        for i, (y, w) in enumerate(zip(ys, want)):
            assert np.array_equal(y.to_host(), w), (rep, i, Ms[i], ctx.last_kernel())
    if K <= 4096:
        assert ctx.last_kernel().startswith("qmv_batch"), ctx.last_kernel()
    for h in xs + ys + [b for l in layers for b in l]:
        h.free()


def test_batch_of_many_items_and_fp32_output(ctx, oracle):
    """More items than one launch takes (48), and fp32 results."""
    K, N, bits, group, n = 1024, 256, 4, 64, 60
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=7, layer=99)
    bw, bs, bb = ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    Ms = [1 + (i % 8) for i in range(n)]
    xh = [oracle.make_x(M, K, oracle.BF16, config_id=7, layer=i, tag=M) for i, M in enumerate(Ms)]
    xs = [ctx.upload(x) for x in xh]
    ys = [ctx.empty((M, N), np.float32) for M in Ms]
    ctx.qmatmul_batch(xs, [bw] * n, [bs] * n, [bb] * n, ys, Ms, K, N, bits, group, F32)
    ref = ctx.empty((8, N), np.float32)
    for i in (0, 7, 47, 48, 59):
        ctx.qmatmul(xs[i], bw, bs, bb, ref, Ms[i], K, N, bits, group, BF16, BF16, F32)
        assert np.array_equal(ys[i].to_host(), ref.to_host((Ms[i], N), np.float32)), i
    for h in xs + ys + [bw, bs, bb, ref]:
        h.free()


def test_dispatch_rereads_its_parameter_buffer_only_when_it_changed(ctx, plugin, oracle):
    """kernel_dispatch takes the shape from a device buffer (the dispatch ABI has no scalars).  The same parameter
    buffer dispatched again is not read back again, and a buffer rewritten in between is: the second shape must
    be the one that runs."""
    import ctypes as C
    from mlx_b200 import plugin as P
    K, N, bits, group = 1024, 256, 4, 64
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=7, layer=1)
    x = oracle.make_x(8, K, oracle.BF16, config_id=7, tag=1)
    bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    y = ctx.empty((8, N), np.uint16)
    v = plugin.vtbl
    k = v.kernel_load(ctx.handle, None, P.QMM_KERNEL_NAME)
    assert k
    prm = P.QmmParams(8, K, N, bits, group, BF16, BF16, BF16)
    pb = v.buffer_alloc_with_data(ctx.handle, C.addressof(prm), C.sizeof(prm))
    bufs = (C.c_void_p * 6)(bx.handle, bw.handle, bs.handle, bb.handle, y.handle, pb)
    want8 = ctx.empty((8, N), np.uint16)
    ctx.qmatmul(bx, bw, bs, bb, want8, 8, K, N, bits, group, BF16, BF16, BF16)
    for _ in range(3):
        plugin.check(v.kernel_dispatch(ctx.handle, k, 0, 0, 0, 0, 0, 0, bufs, 6), "kernel_dispatch")
    assert np.array_equal(y.to_host(), want8.to_host())
    # rewrite the parameters in place: 3 rows of x now; rows 3..7 of y must stay as they are
    prm3 = P.QmmParams(3, K, N, bits, group, BF16, BF16, BF16)
    plugin.check(v.buffer_copy_from_host(ctx.handle, pb, C.addressof(prm3), C.sizeof(prm3)), "copy_from_host")
    marker = np.full((8, N), 0x7FC0, np.uint16)
    y.from_host(marker)
    plugin.check(v.kernel_dispatch(ctx.handle, k, 0, 0, 0, 0, 0, 0, bufs, 6), "kernel_dispatch")
    got = y.to_host()
    assert np.array_equal(got[:3], want8.to_host()[:3]) and np.array_equal(got[3:], marker[3:])
    v.buffer_free(ctx.handle, pb)
    v.kernel_destroy(ctx.handle, k)
    for h in (bx, bw, bs, bb, y, want8):
        h.free()
