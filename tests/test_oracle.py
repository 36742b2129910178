"""The oracle against its pins: hand-computable known answers, the committed
golden fixtures (whose matmul outputs were produced by the reference's own CPU
backend), and -- when the compiled reference is present -- the reference itself."""
import glob
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = sorted(p for p in glob.glob(os.path.join(GOLDEN, "*.npz")) if not p.endswith("kat_words.npz"))


def test_kat_words(oracle):
    k = np.load(os.path.join(GOLDEN, "kat_words.npz"))
    assert np.array_equal(oracle.unpack(k["w4"], 32, 4), k["q4"])
    assert np.array_equal(oracle.unpack(k["w8"], 8, 8), k["q8"])
    assert np.array_equal(oracle.pack(k["q4"], 4), k["w4"])
    assert np.array_equal(oracle.pack(k["q8"], 8), k["w8"])


def test_kat_dequant_identity_and_affine(oracle):
    # s=1, b=0: w^ = q ; s=0.5, b=-4: w^ = q/2 - 4 (all exact in bf16 and fp32)
    q = (np.arange(64, dtype=np.uint8) % 16).reshape(1, 64)
    wq = oracle.pack(q, 4)
    for dt in (oracle.F32, oracle.BF16):
        mk = (lambda v: np.full((1, 1), v, np.float32)) if dt == oracle.F32 else (lambda v: oracle.to_bf16(np.full((1, 1), v, np.float32)))
        w = oracle.dequantize(wq, mk(1.0), mk(0.0), 64, 4, 64, dt)
        wf = w if dt == oracle.F32 else oracle.from_bf16(w)
        assert np.array_equal(wf, q.astype(np.float32))
        w = oracle.dequantize(wq, mk(0.5), mk(-4.0), 64, 4, 64, dt)
        wf = w if dt == oracle.F32 else oracle.from_bf16(w)
        assert np.array_equal(wf, q.astype(np.float32) * 0.5 - 4.0)


def test_bf16_dequant_is_single_rounding(oracle):
    # against an independent computation: exact double arithmetic, one RNE to bf16 (via torch)
    import torch
    wq, s, b = oracle.make_layer(32, 256, 8, 128, oracle.BF16, config_id=7)
    b = oracle.to_bf16(oracle.from_bf16(b) * 1.37)  # break the bias = -128*scale relation
    w = oracle.dequantize(wq, s, b, 256, 8, 128, oracle.BF16)
    q = oracle.unpack(wq, 256, 8).astype(np.float64)
    sf = np.repeat(oracle.from_bf16(s).astype(np.float64), 128, axis=1)
    bf = np.repeat(oracle.from_bf16(b).astype(np.float64), 128, axis=1)
    exact = torch.from_numpy(sf * q + bf).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(exact, w)


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[:-4] for p in CASES])
def test_golden(oracle, path):
    g = np.load(path)
    M, K, N, bits, group, dt = (int(g[k]) for k in ("M", "K", "N", "bits", "group", "dtype"))
    assert np.array_equal(oracle.unpack(g["wq"], K, bits), g["q"])
    assert np.array_equal(oracle.pack(g["q"], bits), g["wq"])
    assert np.array_equal(oracle.dequantize(g["wq"], g["scales"], g["biases"], K, bits, group, dt), g["w"])
    y = oracle.qmatmul_ref(g["x"], g["wq"], g["scales"], g["biases"], bits, group, y_dtype=oracle.F32)
    # bit-exact with what the reference CPU backend computed from the same dequantised weights
    assert np.array_equal(y, g["y_refcore"])
    assert np.array_equal(oracle.qmatmul_ref_rowcache(g["x"], g["wq"], g["scales"], g["biases"], bits, group, y_dtype=oracle.F32), y)
    t = oracle.qmatmul_truth(g["x"], g["wq"], g["scales"], g["biases"], bits, group)
    assert np.array_equal(t, g["truth"])
    err, nerr = oracle.rel_err(y, t)
    assert nerr <= oracle.TOL[dt]


def test_oracle_vs_compiled_reference(oracle):
    """Live pin (only where oracle/_ref was built): the reference's dense fp32
    matmul on dequantised weights equals the oracle's fused quantized matmul."""
    from oracle import refcore
    if not refcore.available():
        pytest.skip("oracle/_ref not built on this machine")
    rc = refcore.RefCore()
    try:
        wq, s, b = oracle.make_layer(96, 512, 4, 64, oracle.F32, config_id=11, bias_noise=1e-3)
        x = oracle.make_x(4, 512, oracle.F32, config_id=11)
        w = oracle.dequantize(wq, s, b, 512, 4, 64, oracle.F32)
        assert np.array_equal(rc.matmul(x, np.ascontiguousarray(w.T)), oracle.qmatmul_ref(x, wq, s, b, 4, 64))
        a = oracle.gen_normal(5, (7, 33))
        bm = oracle.gen_normal(6, (33, 9))
        assert np.array_equal(rc.matmul(a, bm), oracle.matmul_f32(a, bm))
    finally:
        rc.close()


def test_edge_shapes(oracle):
    # empty M, N; K = one group; M=1 row equals the matching row of an M=16 run
    wq, s, b = oracle.make_layer(8, 64, 4, 64, oracle.BF16, config_id=3)
    x = oracle.make_x(16, 64, oracle.BF16, config_id=3)
    y16 = oracle.qmatmul_ref(x, wq, s, b, 4, 64)
    for m in (0, 5, 15):
        assert np.array_equal(oracle.qmatmul_ref(x[m:m + 1], wq, s, b, 4, 64), y16[m:m + 1])
    assert oracle.qmatmul_ref(x[:0], wq, s, b, 4, 64).shape == (0, 8)
    assert oracle.qmatmul_ref(x, wq[:0], s[:0], b[:0], 4, 64).shape == (16, 0)
    with pytest.raises(ValueError):
        oracle.qmatmul_ref(x, wq, oracle.from_bf16(s), oracle.from_bf16(b), 4, 64)  # bf16 x needs bf16 scales
    with pytest.raises(ValueError):
        oracle.qmatmul_ref(x, wq, s, b, 4, 48)  # K not a multiple of group


def test_quantize_roundtrip(oracle):
    w = oracle.gen_normal(99, (16, 256), 0.0, 0.05)
    for bits, group in ((4, 64), (8, 128), (4, 32)):
        wq, s, b = oracle.quantize(w, bits, group, oracle.F32)
        wd = oracle.dequantize(wq, s, b, 256, bits, group, oracle.F32)
        step = np.repeat(s, group, axis=1)
        assert np.all(np.abs(wd - w) <= 0.5 * step * 1.001 + 1e-7)
        # idempotent: quantising the dequantised weights reproduces the codes
        wq2, _, _ = oracle.quantize(wd, bits, group, oracle.F32)
        assert np.mean(oracle.unpack(wq2, 256, bits) == oracle.unpack(wq, 256, bits)) > 0.99


def test_rms_norm(oracle):
    x = oracle.gen_normal(5, (3, 128))
    y = oracle.rms_norm(x, eps=1e-6)
    ref = x / np.sqrt(np.mean(x.astype(np.float64) ** 2, axis=1, keepdims=True) + 1e-6)
    assert np.allclose(y, ref, rtol=1e-5, atol=1e-6)


def test_generators_are_seeded(oracle):
    a = oracle.gen_q(oracle.seed(1, 2), 4, 64, 4)
    assert np.array_equal(a, oracle.gen_q(oracle.seed(1, 2), 4, 64, 4))
    assert not np.array_equal(a, oracle.gen_q(oracle.seed(1, 3), 4, 64, 4))
    wq, s, b = oracle.make_layer(64, 4096, 4, 64, oracle.BF16, config_id=2)
    sf = oracle.from_bf16(s)
    assert sf.min() >= 0.001 * 0.99 and sf.max() <= 0.02 * 1.01
    assert np.array_equal(oracle.from_bf16(b), -8.0 * sf)
    q = oracle.unpack(wq, 4096, 4)
    assert q.min() == 0 and q.max() == 15 and abs(q.mean() - 7.5) < 0.05
    assert oracle.alg_bytes(1, 4096, 11008, 4, 64, 2, 2, 2) == 25392640
    assert oracle.alg_bytes(1, 4096, 4096, 4, 64, 4, 4, 4) == 10518528


def test_chain_elementwise_steps(oracle):
    """The two elementwise steps of the chain configuration, restated with numpy in the oracle: checked against a
    direct scalar evaluation on a small case."""
    rng = np.random.default_rng(3)
    rows, cols = 3, 40
    a = oracle.to_bf16(rng.standard_normal((rows, 3 * cols)).astype(np.float32))
    f = oracle.from_bf16(a)
    want = np.empty((rows, cols), np.float32)
    for r in range(rows):
        for c in range(cols):
            want[r, c] = np.float32(np.float32(f[r, c] + f[r, cols + c]) + f[r, 2 * cols + c])
    assert np.array_equal(oracle.sum3(a, cols), oracle.to_bf16(want))
    m = oracle.to_bf16((f[:, :cols] * f[:, cols:2 * cols]).astype(np.float32))
    got = oracle.mul_rms_norm(a, cols, eps=1e-6)
    assert np.array_equal(got, oracle.rms_norm(m, eps=1e-6))
    mf = oracle.from_bf16(m).astype(np.float64)
    ref = mf / np.sqrt((mf * mf).mean(axis=1, keepdims=True) + 1e-6)
    assert np.abs(oracle.from_bf16(got) - ref).max() <= 2.0 ** -7 * np.abs(ref).max()
