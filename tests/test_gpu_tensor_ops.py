"""The remaining fp32 tensor ops of the base vtable (transpose, reductions, softmax, unary maps, copy,
layer-norm, rms-norm), called through the vtable slots the core forwards to (src/gpu_core.cpp:430-789), against
numpy restatements of the reference's CPU kernels (kernels/cpu/tensor_ops.c).  Elementwise maps and data
movement are exact or within a few fp32 steps of the library functions; reductions within summation-order error."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call(ctx, slot, *args):
    f = getattr(ctx.plugin.vtbl, slot)
    assert f, f"{slot} is NULL"
    ctx.plugin.check(f(ctx.handle, *args), slot)


def _rand(shape, seed, lo=-3.0, hi=3.0):
    return np.random.default_rng(seed).uniform(lo, hi, size=shape).astype(np.float32)


UNARY = {
    "op_exp_f32": (np.exp, (-5, 5)), "op_log_f32": (np.log, (0.01, 50)), "op_sqrt_f32": (np.sqrt, (0, 50)),
    "op_neg_f32": (np.negative, (-3, 3)), "op_abs_f32": (np.abs, (-3, 3)), "op_tanh_f32": (np.tanh, (-4, 4)),
    "op_sigmoid_f32": (lambda x: 1.0 / (1.0 + np.exp(-x)), (-8, 8)), "op_relu_f32": (lambda x: np.maximum(x, 0), (-3, 3)),
    "op_gelu_f32": (lambda x: 0.5 * x * (1.0 + np.tanh(np.float32(0.7978845608) * (x + np.float32(0.044715) * x * x * x))), (-4, 4)),
    "op_copy_f32": (lambda x: x, (-3, 3)),
}


@pytest.mark.parametrize("slot", sorted(UNARY))
def test_unary(ctx, slot):
    fn, (lo, hi) = UNARY[slot]
    n = 100003
    x = _rand((n,), 1, lo, hi)
    bi, bo = ctx.upload(x), ctx.empty((n,), np.float32)
    _call(ctx, slot, bi.handle, bo.handle, n)
    y = bo.to_host()
    want = fn(x.astype(np.float64)).astype(np.float32) if slot not in ("op_copy_f32", "op_neg_f32", "op_abs_f32", "op_relu_f32") else fn(x)
    if slot in ("op_copy_f32", "op_neg_f32", "op_abs_f32", "op_relu_f32", "op_sqrt_f32"):
        assert np.array_equal(y, want.astype(np.float32))
    else:
        assert np.abs(y - want).max() <= 4e-6 * max(1.0, np.abs(want).max())
    bi.free(); bo.free()


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 70), (65, 33), (256, 1000)])
def test_transpose(ctx, rows, cols):
    x = _rand((rows, cols), 2)
    bi, bo = ctx.upload(x), ctx.empty((cols, rows), np.float32)
    _call(ctx, "op_transpose_f32", bi.handle, bo.handle, rows, cols)
    assert np.array_equal(bo.to_host(), x.T)
    bi.free(); bo.free()


@pytest.mark.parametrize("n", [1, 31, 4097, 300000])
def test_full_reductions(ctx, n):
    x = _rand((n,), 3)
    bi, bo = ctx.upload(x), ctx.empty((1,), np.float32)
    for slot, fn, exact in (("op_reduce_sum_f32", np.sum, False), ("op_reduce_max_f32", np.max, True),
                            ("op_reduce_min_f32", np.min, True), ("op_reduce_mean_f32", np.mean, False)):
        _call(ctx, slot, bi.handle, bo.handle, n)
        got, want = float(bo.to_host()[0]), float(fn(x.astype(np.float64)))
        if exact:
            assert got == want
        else:
            assert abs(got - want) <= 1e-5 * np.abs(x).sum() / (n if slot.endswith("mean_f32") else 1) + 1e-6
    bi.free(); bo.free()


def test_axis_reductions(ctx):
    outer, inner = 37, 1234
    x = _rand((outer, inner), 4)
    bi, bo = ctx.upload(x), ctx.empty((outer,), np.float32)
    _call(ctx, "op_reduce_sum_axis_f32", bi.handle, bo.handle, outer, inner)
    assert np.abs(bo.to_host() - x.astype(np.float64).sum(axis=1)).max() <= 1e-3
    _call(ctx, "op_reduce_max_axis_f32", bi.handle, bo.handle, outer, inner)
    assert np.array_equal(bo.to_host(), x.max(axis=1))
    bi.free(); bo.free()


@pytest.mark.parametrize("batch,dim", [(1, 1), (8, 100), (5, 5000)])
def test_softmax_and_log_softmax(ctx, batch, dim):
    x = _rand((batch, dim), 5, -10, 10)
    bi, bo = ctx.upload(x), ctx.empty((batch, dim), np.float32)
    x64 = x.astype(np.float64)
    e = np.exp(x64 - x64.max(axis=1, keepdims=True))
    _call(ctx, "op_softmax_f32", bi.handle, bo.handle, batch, dim)
    y = bo.to_host()
    assert np.abs(y - e / e.sum(axis=1, keepdims=True)).max() <= 1e-6
    assert np.abs(y.sum(axis=1) - 1.0).max() <= 1e-5
    _call(ctx, "op_log_softmax_f32", bi.handle, bo.handle, batch, dim)
    want = x64 - x64.max(axis=1, keepdims=True) - np.log(e.sum(axis=1, keepdims=True))
    assert np.abs(bo.to_host() - want).max() <= 1e-5
    bi.free(); bo.free()


def test_layer_norm_and_rms_norm(ctx):
    batch, dim, eps = 6, 777, 1e-5
    x, gamma, beta = _rand((batch, dim), 6), _rand((dim,), 7, 0.5, 1.5), _rand((dim,), 8, -0.2, 0.2)
    bi, bo, bg, bb = ctx.upload(x), ctx.empty((batch, dim), np.float32), ctx.upload(gamma), ctx.upload(beta)
    _call(ctx, "op_layer_norm_f32", bi.handle, bo.handle, bg.handle, bb.handle, batch, dim, eps)
    x64 = x.astype(np.float64)
    mean, var = x64.mean(axis=1, keepdims=True), x64.var(axis=1, keepdims=True)
    assert np.abs(bo.to_host() - ((x64 - mean) / np.sqrt(var + eps) * gamma + beta)).max() <= 1e-5
    _call(ctx, "op_rms_norm_f32", bi.handle, bo.handle, bg.handle, batch, dim, eps)
    assert np.abs(bo.to_host() - x64 / np.sqrt((x64 * x64).mean(axis=1, keepdims=True) + eps) * gamma).max() <= 1e-5
    for h in (bi, bo, bg, bb):
        h.free()
