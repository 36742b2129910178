"""The plugin as a drop-in backend of the unmodified reference core: base
vtable semantics through the C ABI, and the reference's own test program
(test/test_core.cpp, built into oracle/_ref by oracle/Makefile) run with
LUX_GPU_BACKEND_PATH pointing at the plugin -- the way its CTest sets it
(CMakeLists.txt:130-132)."""
import os
import subprocess

import numpy as np
import pytest

from mlx_b200 import plugin as P

pytestmark = pytest.mark.gpu
GOLDILOCKS = 0xFFFFFFFF00000001


def test_device_info_and_count(plugin, ctx):
    assert plugin.device_count() >= 1
    info = ctx.device_info()
    assert b"B200" in info.name and info.vendor == b"NVIDIA"
    assert info.compute_units == 148 and info.is_discrete and not info.is_unified_memory
    assert info.memory_total > 100 << 30


def test_buffers(ctx):
    z = ctx.alloc(1 << 20, (1 << 18,), np.float32)
    assert not z.to_host().any()  # buffer_alloc zero-fills like the CPU backend (src/cpu_backend.cpp:129)
    a = np.arange(1000, dtype=np.float32)
    b = ctx.upload(a)
    assert np.array_equal(b.to_host(), a)
    # copies clamp to the buffer size (src/cpu_backend.cpp:151,158)
    big = np.empty(2000, np.float32); big[:] = -1
    ctx.plugin.check(ctx.plugin.vtbl.buffer_copy_to_host(ctx.handle, b.handle, big.ctypes.data, big.nbytes), "copy")
    assert np.array_equal(big[:1000], a) and (big[1000:] == -1).all()
    b.from_host(a[::-1].copy())
    assert np.array_equal(b.to_host(), a[::-1])
    assert ctx.plugin.vtbl.buffer_get_host_ptr(ctx.handle, b.handle) is None
    z.free(); b.free()


def test_allocator_caches_and_reuses(ctx):
    s0 = ctx.allocator_stats()
    for _ in range(50):
        t = ctx.alloc(3 << 20)
        t.free()
    s1 = ctx.allocator_stats()
    assert s1["driver_allocs"] - s0["driver_allocs"] <= 1  # 50 alloc/free cycles, at most one cudaMalloc
    assert s1["in_use"] == s0["in_use"]


def test_buffer_outlives_context(plugin):
    """The core destroys a context before the tensors made on it
    (src/gpu_core.cpp:216-233); buffer_free must still work."""
    c = plugin.context(0)
    b = c.upload(np.ones(16, np.float32))
    h = c.handle
    c.close()
    plugin.vtbl.buffer_free(h, b.handle)  # dangling ctx pointer is ignored
    b.handle = None


def test_elementwise_and_matmul_match_reference_cpu_backend(ctx, oracle):
    a = oracle.gen_normal(1, (1000,)); b = oracle.gen_normal(2, (1000,)) + 3.0
    ba, bb, bo = ctx.upload(a), ctx.upload(b), ctx.empty((1000,), np.float32)
    for op, f in (("add", np.add), ("sub", np.subtract), ("mul", np.multiply), ("div", np.divide)):
        ctx.binary(op, ba, bb, bo, 1000)
        assert np.array_equal(bo.to_host(), f(a, b))
    # the harness's 2x2 case (test/test_core.cpp:93-117)
    A = np.array([[1, 2], [3, 4]], np.float32); B = np.array([[5, 6], [7, 8]], np.float32)
    bA, bB, bC = ctx.upload(A), ctx.upload(B), ctx.empty((2, 2), np.float32)
    ctx.matmul_f32(bA, bB, bC, 2, 2, 2)
    assert np.array_equal(bC.to_host(), np.array([[19, 22], [43, 50]], np.float32))
    # bit-identical to the CPU backend's sequential fp32 sum (src/cpu_backend.cpp:253-264)
    A = oracle.gen_normal(3, (37, 300)); B = oracle.gen_normal(4, (300, 53))
    bA2, bB2, bC2 = ctx.upload(A), ctx.upload(B), ctx.empty((37, 53), np.float32)
    ctx.matmul_f32(bA2, bB2, bC2, 37, 300, 53)
    assert np.array_equal(bC2.to_host(), oracle.matmul_f32(A, B))
    for h in (ba, bb, bo, bA, bB, bC, bA2, bB2, bC2):
        h.free()


def test_ntt_roundtrip_and_known_values(ctx):
    d = np.arange(1, 9, dtype=np.uint64)
    f = ctx.ntt(d.copy(), GOLDILOCKS)
    assert int(f[0]) == 36  # sum of the inputs
    assert np.array_equal(ctx.ntt(f.copy(), GOLDILOCKS, inverse=True), d)
    rng = np.random.default_rng(0)
    for n in (1, 2, 64, 4096):
        d = rng.integers(0, GOLDILOCKS, n, dtype=np.uint64)
        assert np.array_equal(ctx.ntt(ctx.ntt(d.copy(), GOLDILOCKS), GOLDILOCKS, inverse=True), d)
    with pytest.raises(P.BackendError):
        ctx.ntt(np.zeros(6, np.uint64), GOLDILOCKS)  # not a power of two


def test_reference_harness_runs_on_the_plugin():
    from oracle import refcore
    if not os.path.exists(refcore.TEST_CORE_BIN):
        pytest.skip("oracle/_ref/test_gpu_core was not built")
    env = dict(os.environ, LUX_GPU_BACKEND_PATH=os.path.dirname(P.LIB_PATH))
    r = subprocess.run([refcore.TEST_CORE_BIN], env=env, capture_output=True, text=True, timeout=300)
    print(r.stdout)
    assert "(cuda)" in r.stdout, r.stdout  # AUTO picked our plugin, not the CPU fallback
    assert "Failed: 0" in r.stdout and "Passed: 17" in r.stdout and r.returncode == 0


def test_reference_public_api_on_the_plugin(oracle):
    """lux_tensor_matmul through the unmodified core, backend = our plugin."""
    from oracle import refcore
    if not refcore.available():
        pytest.skip("oracle/_ref not built")
    os.environ["LUX_GPU_BACKEND_PATH"] = os.path.dirname(P.LIB_PATH)
    rc = refcore.RefCore(backend=refcore.BACKEND_CUDA)
    try:
        assert rc.backend_name == "cuda"
        A = oracle.gen_normal(3, (5, 64)); B = oracle.gen_normal(4, (64, 7))
        assert np.array_equal(rc.matmul(A, B), oracle.matmul_f32(A, B))
        assert np.array_equal(rc.binary("add", A, A), A + A)
    finally:
        rc.close()


def test_allocation_failure_is_a_null_buffer_with_a_message(plugin, ctx):
    """A request beyond the device's memory comes back as NULL (the reference's convention for a failed
    buffer_alloc, src/cpu_backend.cpp:121-131) with an out-of-memory text, and the context stays usable."""
    info = ctx.device_info()
    too_much = int(info.memory_total) * 4 if getattr(info, "memory_total", 0) else (1 << 42)
    h = plugin.vtbl.buffer_alloc(ctx.handle, too_much)
    assert not h
    msg = plugin.last_error().lower()
    assert "memory" in msg, msg
    b = ctx.upload(np.arange(8, dtype=np.float32))   # still works
    assert np.array_equal(b.to_host(), np.arange(8, dtype=np.float32))
    b.free()
