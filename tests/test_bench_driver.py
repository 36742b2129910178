"""The C host loops of bench.py's end-to-end leg (bench_e2e.c), driven with fake entry points on the CPU: order of
the calls, counts, and that a failing call ends the loop with its code."""
import ctypes as C
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402

COPY_IN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t)
COPY_OUT = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t)
BATCH = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                    C.c_int, C.c_int, C.c_int, C.c_int, C.c_int)
PUSH_BATCH = BATCH


class Batch(C.Structure):
    _fields_ = [("x_all_dev", C.c_void_p), ("x_all_host", C.c_void_p), ("x_bytes", C.c_size_t),
                ("y_all_dev", C.c_void_p), ("y_all_host", C.c_void_p), ("y_bytes", C.c_size_t), ("n", C.c_int32),
                ("x", C.c_void_p), ("wq", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p), ("y", C.c_void_p),
                ("y_offset", C.c_void_p), ("M", C.c_void_p), ("y_symm", C.c_void_p),
                ("K", C.c_int32), ("N", C.c_int32), ("bits", C.c_int32), ("group", C.c_int32), ("dtype", C.c_int32)]


def driver():
    drv = C.CDLL(bench.e2e_driver_path())
    drv.lux_bench_e2e_batch.restype = C.c_int
    drv.lux_bench_e2e_batch.argtypes = [C.c_void_p] * 5 + [C.POINTER(Batch), C.c_int, C.POINTER(C.c_longlong)]
    drv.lux_bench_e2e_batch2.restype = C.c_int
    drv.lux_bench_e2e_batch2.argtypes = [C.c_void_p] * 3 + [C.POINTER(C.c_void_p), C.POINTER(C.POINTER(Batch)), C.c_int,
                                                            C.POINTER(C.c_longlong)]
    return drv


def fakes(log, fail_at=None):
    def step(tag, ctx):
        log.append((tag, ctx))
        return 7 if fail_at is not None and len(log) == fail_at else 0
    cin = COPY_IN(lambda ctx, buf, src, n: step("in", ctx))
    cout = COPY_OUT(lambda ctx, buf, dst, n: step("out", ctx))
    bat = BATCH(lambda ctx, n, *a: step("batch", ctx))
    push = PUSH_BATCH(lambda sb, n, *a: step("push", sb))
    return cin, cout, bat, push


def test_one_context_loop_order_and_error():
    drv = driver()
    log = []
    cin, cout, bat, push = fakes(log)
    b = Batch(n=48, y_symm=None)
    done = C.c_longlong(0)
    addr = lambda f: C.cast(f, C.c_void_p)
    assert drv.lux_bench_e2e_batch(addr(cin), addr(bat), addr(push), addr(cout), 11, C.byref(b), 3, C.byref(done)) == 0
    assert [t for t, _ in log] == ["in", "batch", "out"] * 3 and done.value == 3 * 48
    log.clear()
    b.y_symm = 99  # sharded: the batched push is called with the symmetric buffer, not the context
    assert drv.lux_bench_e2e_batch(addr(cin), addr(bat), addr(push), addr(cout), 11, C.byref(b), 2, C.byref(done)) == 0
    assert log == [("in", 11), ("push", 99), ("out", 11)] * 2
    log.clear()
    cin, cout, bat, push = fakes(log, fail_at=5)
    assert drv.lux_bench_e2e_batch(addr(cin), addr(bat), addr(push), addr(cout), 11, C.byref(b), 3, C.byref(done)) == 7
    assert len(log) == 5


def test_two_context_loop_keeps_one_sweep_in_flight():
    drv = driver()
    log = []
    cin, cout, bat, _ = fakes(log)
    b0, b1 = Batch(n=5), Batch(n=5)
    ctxs = (C.c_void_p * 2)(100, 200)
    bs = (C.POINTER(Batch) * 2)(C.pointer(b0), C.pointer(b1))
    done = C.c_longlong(0)
    addr = lambda f: C.cast(f, C.c_void_p)
    assert drv.lux_bench_e2e_batch2(addr(cin), addr(bat), addr(cout), ctxs, bs, 4, C.byref(done)) == 0
    assert done.value == 20
    # sweep r is enqueued on context r % 2 before sweep r-1 is read back from the other one
    assert log == [("in", 100), ("batch", 100),
                   ("in", 200), ("batch", 200), ("out", 100),
                   ("in", 100), ("batch", 100), ("out", 200),
                   ("in", 200), ("batch", 200), ("out", 100),
                   ("out", 200)]
