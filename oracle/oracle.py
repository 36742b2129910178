"""ctypes/numpy front end of ``qmm_oracle.c`` (test infrastructure only).

bf16 tensors are carried as ``numpy.uint16`` arrays holding the raw bits.
dtype codes follow include/lux/gpu/backend_plugin.h:38-47 (F32 = 0, BF16 = 2).
"""
import ctypes as C
import os
import subprocess

import numpy as np

F32, BF16, U32 = 0, 2, 5
BASE_SEED = 20261125

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

__all__ = [
    "F32", "BF16", "U32", "BASE_SEED", "build", "lib", "seed", "gen_q", "gen_uniform", "gen_normal",
    "to_bf16", "from_bf16", "unpack", "pack", "dequantize", "qmatmul_ref", "qmatmul_ref_rowcache",
    "qmatmul_truth", "matmul_f32", "rms_norm", "sum3", "mul_rms_norm", "quantize", "num_threads", "set_num_threads",
    "make_layer", "make_x", "rel_err", "REL_FLOOR", "alg_bytes", "TOL",
]

# tolerances of the path (north_star): max relative error, by compute dtype
TOL = {BF16: 1e-2, F32: 1e-4}


def _reference_root():
    """The reference tree: $REF, else a directory ``reference`` beside this repository or beside a directory above it."""
    env = os.environ.get("REF")
    if env:
        return env if os.path.isdir(env) else None
    d = os.path.dirname(os.path.realpath(_HERE))
    while True:
        parent = os.path.dirname(d)
        if parent == d:
            return None
        cand = os.path.join(parent, "reference")
        if os.path.exists(os.path.join(cand, "src", "gpu_core.cpp")):
            return cand
        d = parent


def build(force=False):
    """Compile the oracle (and the reference core when its tree is present)."""
    src = os.path.join(_HERE, "qmm_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    ref = _reference_root()
    if force or stale or (ref and not os.path.exists(os.path.join(_HERE, "_ref", "test_gpu_core"))):
        subprocess.run(["make", "-C", _HERE, "all"] + ([f"REF={ref}"] if ref else []), check=True, stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_seed.restype = C.c_uint64
        _lib.orc_seed.argtypes = [C.c_uint64] * 5
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def seed(*ids, base=BASE_SEED):
    ids = list(ids) + [0] * (4 - len(ids))
    return int(lib().orc_seed(base, *[int(i) & (2**64 - 1) for i in ids]))


def gen_q(sd, N, K, bits):
    out = np.empty((N, K * bits // 32), dtype=np.uint32)
    lib().orc_gen_q(C.c_uint64(sd), _p(out), C.c_int64(N), C.c_int64(K), C.c_int(bits))
    return out


def gen_uniform(sd, shape, lo, hi):
    out = np.empty(shape, dtype=np.float32)
    lib().orc_gen_uniform_f32(C.c_uint64(sd), _p(out), C.c_int64(out.size), C.c_double(lo), C.c_double(hi))
    return out


def gen_normal(sd, shape, mean=0.0, std=1.0):
    out = np.empty(shape, dtype=np.float32)
    lib().orc_gen_normal_f32(C.c_uint64(sd), _p(out), C.c_int64(out.size), C.c_double(mean), C.c_double(std))
    return out


def to_bf16(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    out = np.empty(a.shape, dtype=np.uint16)
    lib().orc_round_bf16(_p(a), _p(out), C.c_int64(a.size))
    return out


def from_bf16(a):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, dtype=np.float32)
    lib().orc_widen_bf16(_p(a), _p(out), C.c_int64(a.size))
    return out


def _dt(a):
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.uint16:
        return BF16
    raise TypeError(f"unsupported dtype {a.dtype}")


def unpack(wq, K, bits):
    wq = np.ascontiguousarray(wq, dtype=np.uint32)
    N = wq.shape[0]
    out = np.empty((N, K), dtype=np.uint8)
    lib().orc_unpack(_p(wq), _p(out), C.c_int64(N), C.c_int64(K), C.c_int(bits))
    return out


def pack(q, bits):
    q = np.ascontiguousarray(q, dtype=np.uint8)
    N, K = q.shape
    out = np.empty((N, K * bits // 32), dtype=np.uint32)
    lib().orc_pack(_p(q), _p(out), C.c_int64(N), C.c_int64(K), C.c_int(bits))
    return out


def dequantize(wq, scales, biases, K, bits, group, out_dtype):
    N = wq.shape[0]
    out = np.empty((N, K), dtype=np.uint16 if out_dtype == BF16 else np.float32)
    rc = lib().orc_dequantize(_p(wq), _p(scales), _p(biases), _p(out), C.c_int64(N), C.c_int64(K),
                              C.c_int(bits), C.c_int(group), C.c_int(_dt(scales)), C.c_int(out_dtype))
    if rc:
        raise ValueError(f"orc_dequantize rc={rc}")
    return out


def _qmm(fn, x, wq, scales, biases, bits, group, y_dtype):
    x = np.ascontiguousarray(x)
    M, K = x.shape
    N = wq.shape[0]
    y = np.empty((M, N), dtype=np.uint16 if y_dtype == BF16 else np.float32)
    rc = fn(_p(x), _p(wq), _p(scales), _p(biases), _p(y), C.c_int64(M), C.c_int64(K), C.c_int64(N),
            C.c_int(bits), C.c_int(group), C.c_int(_dt(x)), C.c_int(_dt(scales)), C.c_int(y_dtype))
    if rc:
        raise ValueError(f"oracle qmatmul rc={rc}")
    return y


def qmatmul_ref(x, wq, scales, biases, bits, group, y_dtype=None):
    """Reference-style (collapse(2), sequential fp32 k-sum) quantized matmul."""
    return _qmm(lib().orc_qmatmul_ref, x, wq, scales, biases, bits, group, _dt(x) if y_dtype is None else y_dtype)


def qmatmul_ref_rowcache(x, wq, scales, biases, bits, group, y_dtype=None):
    return _qmm(lib().orc_qmatmul_ref_rowcache, x, wq, scales, biases, bits, group,
                _dt(x) if y_dtype is None else y_dtype)


def qmatmul_truth(x, wq, scales, biases, bits, group):
    x = np.ascontiguousarray(x)
    M, K = x.shape
    N = wq.shape[0]
    y = np.empty((M, N), dtype=np.float64)
    rc = lib().orc_qmatmul_truth(_p(x), _p(wq), _p(scales), _p(biases), _p(y), C.c_int64(M), C.c_int64(K),
                                 C.c_int64(N), C.c_int(bits), C.c_int(group), C.c_int(_dt(x)), C.c_int(_dt(scales)))
    if rc:
        raise ValueError(f"orc_qmatmul_truth rc={rc}")
    return y


def matmul_f32(a, b):
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    M, K = a.shape
    N = b.shape[1]
    out = np.empty((M, N), dtype=np.float32)
    lib().orc_matmul_f32(_p(a), _p(b), _p(out), C.c_int(M), C.c_int(K), C.c_int(N))
    return out


def rms_norm(x, eps=1e-6, weight=None, out_dtype=None):
    x = np.ascontiguousarray(x)
    rows, dim = x.shape
    od = _dt(x) if out_dtype is None else out_dtype
    out = np.empty((rows, dim), dtype=np.uint16 if od == BF16 else np.float32)
    w = None if weight is None else np.ascontiguousarray(weight, dtype=np.float32)
    lib().orc_rms_norm(_p(x), _p(out), _p(w), C.c_int64(rows), C.c_int64(dim), C.c_float(eps),
                       C.c_int(_dt(x)), C.c_int(od))
    return out


def sum3(qkv, cols):
    """bf16(q + k + v) over the three column blocks of a bf16 [rows, >= 3*cols] array: fp32 adds, left to right,
    one rounding (the elementwise add of the reference, src/cpu_backend.cpp:186-203, applied twice)."""
    f = from_bf16(np.ascontiguousarray(qkv))
    s = (f[:, :cols] + f[:, cols:2 * cols]).astype(np.float32) + f[:, 2 * cols:3 * cols]
    return to_bf16(s.astype(np.float32))


def mul_rms_norm(gu, cols, eps=1e-6):
    """rms_norm(bf16(gate * up)) over the two column blocks of a bf16 [rows, >= 2*cols] array (elementwise
    product of the reference, src/cpu_backend.cpp:224-241; rms-norm formula of kernels/cpu/tensor_ops.c:546-566)."""
    f = from_bf16(np.ascontiguousarray(gu))
    m = to_bf16((f[:, :cols] * f[:, cols:2 * cols]).astype(np.float32))
    return rms_norm(m, eps=eps)


def quantize(w, bits, group, sb_dtype):
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    wq = np.empty((N, K * bits // 32), dtype=np.uint32)
    sdt = np.uint16 if sb_dtype == BF16 else np.float32
    s = np.empty((N, K // group), dtype=sdt)
    b = np.empty((N, K // group), dtype=sdt)
    rc = lib().orc_quantize(_p(w), _p(wq), _p(s), _p(b), C.c_int64(N), C.c_int64(K), C.c_int(bits),
                            C.c_int(group), C.c_int(sb_dtype))
    if rc:
        raise ValueError(f"orc_quantize rc={rc}")
    return wq, s, b


def num_threads():
    return int(lib().orc_num_threads())


def set_num_threads(n):
    lib().orc_set_num_threads(C.c_int(int(n)))


# ---------------------------------------------------------------------------
# Seeded synthetic layers in the shapes and distributions of the benchmark
# configurations (these *are* the benchmark inputs; no external dataset).
# ---------------------------------------------------------------------------
def make_layer(N, K, bits, group, sb_dtype, config_id=0, layer=0, proj=0, bias_noise=0.0,
               scale_range=None):
    """Return (wq, scales, biases).  q ~ U{0..2^bits-1}; scales ~ U(range),
    rounded to bf16 first when sb_dtype is BF16; biases = -(2^(bits-1))*scale
    (+ N(0, bias_noise) for the fp32 configuration)."""
    if scale_range is None:
        scale_range = (0.001, 0.02) if bits == 4 else (1e-4, 2e-3)
    wq = gen_q(seed(config_id, 1, layer, proj), N, K, bits)
    s = gen_uniform(seed(config_id, 2, layer, proj), (N, K // group), *scale_range)
    half = float(1 << (bits - 1))
    if sb_dtype == BF16:
        s16 = to_bf16(s)
        b16 = to_bf16(-half * from_bf16(s16))  # exact: power-of-two multiple
        return wq, s16, b16
    b = (-half * s).astype(np.float32)
    if bias_noise:
        b = (b + gen_normal(seed(config_id, 3, layer, proj), b.shape, 0.0, bias_noise)).astype(np.float32)
    return wq, s, b


def make_x(M, K, dtype, config_id=0, layer=0, tag=0):
    x = gen_normal(seed(config_id, 4, layer, tag), (M, K))
    return to_bf16(x) if dtype == BF16 else x


REL_FLOOR = 1e-2


def rel_err(y, truth, floor=REL_FLOOR):
    """(max_i |y_i - t_i| / max(|t_i|, floor * max|t|),  max|y - t| / max|t|).

    The first figure is the "max relative error" the tolerances apply to.
    Outputs that are small only through cancellation cannot hold a relative
    bound in ANY fp32-accumulating implementation, so elements below
    floor * max|t| are measured against that floor.  floor = 1e-2: with 1e-3
    the reference-style sequential fp32 loop itself misses the 1e-4 fp32 bar
    on the 4096x4096 CPU configuration (5.1e-4; 6.3e-5 at 1e-2)."""
    y = from_bf16(y).astype(np.float64) if y.dtype == np.uint16 else y.astype(np.float64)
    t = truth.astype(np.float64)
    tmax = float(np.max(np.abs(t))) if t.size else 0.0
    if t.size == 0 or tmax == 0.0:
        return 0.0, 0.0
    d = np.abs(y - t)
    return float(np.max(d / np.maximum(np.abs(t), floor * tmax))), float(np.max(d) / tmax)


def alg_bytes(M, K, N, bits, group, x_size, sb_size, y_size):
    """Algorithmic bytes of one quantized matmul: every operand exactly once."""
    return N * K * bits // 8 + 2 * (N * K // group) * sb_size + M * K * x_size + M * N * y_size
