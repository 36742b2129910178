"""The allocation-free decode entry point (lux_gpu_cuda_qmatmul_decode_noalloc).

Some hosts cannot let the plugin allocate once they are serving: all of HBM already belongs to
their own arena, or allocation is simply forbidden after start-up.  For them the library carries
a fixed scratch array inside its image.  This test calls that entry point through the C ABI and
requires the same bits as the ordinary qmatmul, twice in a row (the scratch is shared between
calls and must come back clean), including a shape whose K is split over several thread blocks
and therefore really goes through the scratch.  It also checks that the allocator is not touched
and that an over-sized request is refused rather than overrunning the array.

Collected last on purpose: a failure here must not hide the other GPU tests under `-x`.
"""
import numpy as np
import pytest

from mlx_b200 import BF16, F32, BackendError
from mlx_b200 import plugin as P

pytestmark = pytest.mark.gpu

SHAPES = [
    # M, K, N, bits, group
    (1, 4096, 11008, 4, 64),    # the benchmark's decode layer: counters only
    (8, 8192, 64, 4, 64),       # few rows, long K: K is split, partials travel through the scratch
    (16, 4096, 96, 8, 128),     # 8-bit, split
    (3, 1024, 100, 4, 32),
]


@pytest.mark.parametrize("M,K,N,bits,group", SHAPES)
def test_noalloc_matches_qmatmul_twice(ctx, oracle, M, K, N, bits, group):
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=13, layer=K, proj=N)
    x = oracle.make_x(M, K, oracle.BF16, config_id=13, tag=M)
    bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    y_ref = ctx.empty((M, N), np.uint16)
    ctx.qmatmul(bx, bw, bs, bb, y_ref, M, K, N, bits, group, BF16, BF16, BF16)
    want = y_ref.to_host()
    err, _ = oracle.rel_err(want, oracle.qmatmul_truth(x, wq, s, b, bits, group))
    assert err <= oracle.TOL[oracle.BF16]
    before = ctx.allocator_stats()
    y = ctx.empty((M, N), np.uint16)
    after_y = ctx.allocator_stats()
    for call in range(2):
        y.from_host(np.zeros((M, N), np.uint16))
        ctx.qmatmul_decode_noalloc(bx, bw, bs, bb, y, M, K, N, bits, group, BF16)
        assert ctx.last_kernel().startswith("qmv_mma")
        assert np.array_equal(y.to_host(), want), f"call {call}"
    # nothing was taken from the allocator by the calls themselves
    assert ctx.allocator_stats() == after_y and after_y["driver_allocs"] >= before["driver_allocs"]
    # fp32 output goes the same way
    yf_ref, yf = ctx.empty((M, N), np.float32), ctx.empty((M, N), np.float32)
    ctx.qmatmul(bx, bw, bs, bb, yf_ref, M, K, N, bits, group, BF16, BF16, F32)
    ctx.qmatmul_decode_noalloc(bx, bw, bs, bb, yf, M, K, N, bits, group, F32)
    assert np.array_equal(yf.to_host(), yf_ref.to_host())
    for h in (bx, bw, bs, bb, y_ref, y, yf_ref, yf):
        h.free()


def test_noalloc_refuses_what_does_not_fit(ctx, oracle, plugin):
    # 74 row tiles x 64 k-blocks x 16 rows of x: 4.8 MB of partials, more than the built-in 4 MiB
    M, K, N = 16, 16384, 1184
    wq, s, b = oracle.make_layer(N, K, 4, 64, oracle.BF16, config_id=14)
    x = oracle.make_x(M, K, oracle.BF16, config_id=14)
    bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b)
    y = ctx.empty((M, N), np.uint16)
    with pytest.raises(BackendError) as ei:
        ctx.qmatmul_decode_noalloc(bx, bw, bs, bb, y, M, K, N, 4, 64, BF16)
    assert ei.value.code == P.ERR_INVALID and "scratch" in plugin.last_error()
    # the ordinary entry point takes the same shape
    ctx.qmatmul(bx, bw, bs, bb, y, M, K, N, 4, 64, BF16, BF16, BF16)
    err, _ = oracle.rel_err(y.to_host(), oracle.qmatmul_truth(x, wq, s, b, 4, 64))
    assert err <= oracle.TOL[oracle.BF16]
    # shapes outside the decode kernel and bad arguments are errors, not crashes
    with pytest.raises(BackendError) as ei:
        ctx.qmatmul_decode_noalloc(bx, bw, bs, bb, y, 17, K, N, 4, 64, BF16)
    assert ei.value.code == P.ERR_INVALID
    with pytest.raises(BackendError) as ei:
        ctx.qmatmul_decode_noalloc(bx, bw, bs, bb, y, 2, 192, 8, 4, 64, BF16)
    assert ei.value.code == P.ERR_NOT_SUPPORTED
    for h in (bx, bw, bs, bb, y):
        h.free()


def test_noalloc_scratch_shared_between_split_shapes(plugin, ctx, oracle):
    """One scratch array serves every shape: a K-split call with few row tiles, then one with more than 64 row
    tiles (whose arrival counters used to reach into the region where the first call's partials had lain), then
    the first again.  Each must give the bits of the ordinary qmatmul on a fresh context."""
    fresh = plugin.context(0)
    try:
        for (M, K, N, bits, group) in ((8, 8192, 64, 4, 64), (1, 8192, 1120, 4, 64), (8, 8192, 64, 4, 64), (1, 8192, 1120, 4, 64)):
            wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=13, layer=K, proj=N)
            x = oracle.make_x(M, K, oracle.BF16, config_id=13, tag=M)
            fx, fw, fs, fb = fresh.upload(x), fresh.upload(wq), fresh.upload(s), fresh.upload(b)
            y_ref = fresh.empty((M, N), np.uint16)
            fresh.qmatmul(fx, fw, fs, fb, y_ref, M, K, N, bits, group, BF16, BF16, BF16)
            want = y_ref.to_host()
            bx, bw, bs, bb = ctx.upload(x), ctx.upload(wq), ctx.upload(s), ctx.upload(b)
            y = ctx.empty((M, N), np.uint16)
            ctx.qmatmul_decode_noalloc(bx, bw, bs, bb, y, M, K, N, bits, group, BF16)
            assert ctx.last_kernel().startswith("qmv_mma")
            assert np.array_equal(y.to_host(), want), (M, K, N)
            for h in (fx, fw, fs, fb, y_ref, bx, bw, bs, bb, y):
                h.free()
    finally:
        fresh.close()
