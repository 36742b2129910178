"""ctypes mirror of the Lux GPU backend plugin ABI for libluxgpu_backend_cuda.so.

Performs the same three steps as the reference's plugin loader
(src/plugin_loader.hpp:184-232): dlopen, ``lux_gpu_backend_init``, ABI-version
check (== 2, include/lux/gpu/backend_plugin.h:24), and then exposes the base
vtable (backend_plugin.h:82-382) and the quantized-matmul extension table
(include/lux_cuda_quant.h).  There is no CPU fallback here: if the library is
missing or reports no usable GPU, construction raises.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libluxgpu_backend_cuda.so")

ABI_VERSION = 2
F32, F16, BF16, I32, I64, U32, U64, BOOL = range(8)  # backend_plugin.h:38-47
OK, ERR_INVALID, ERR_OOM, ERR_NOT_SUPPORTED, ERR_DEVICE_LOST, ERR_INTERNAL = range(6)  # backend_plugin.h:49-56
ERR_NAMES = ["OK", "INVALID_ARGUMENT", "OUT_OF_MEMORY", "NOT_SUPPORTED", "DEVICE_LOST", "INTERNAL"]
QUANT_MAGIC = 0x4C515854
QMM_KERNEL_NAME = b"lux.qmm.affine"
NCCL_UID_BYTES = 128

_vp, _sz, _i, _u32, _u64 = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_uint64


class DeviceInfo(C.Structure):  # backend_plugin.h:58-67
    _fields_ = [("name", C.c_char_p), ("vendor", C.c_char_p), ("memory_total", _u64), ("memory_available", _u64),
                ("compute_units", _i), ("max_workgroup_size", _i), ("is_discrete", C.c_bool),
                ("is_unified_memory", C.c_bool)]


def _fn(res, *args):
    return C.CFUNCTYPE(res, *args)


_BIN = _fn(_i, _vp, _vp, _vp, _vp, _sz)
_UN = _fn(_i, _vp, _vp, _vp, _sz)

# The 64 slots of lux_gpu_backend_vtbl in declaration order (backend_plugin.h:82-382).
_VTBL_FIELDS = [
    ("create_context", _fn(_vp, _i)),
    ("destroy_context", _fn(None, _vp)),
    ("get_device_count", _fn(_i, C.POINTER(_i))),
    ("get_device_info", _fn(_i, _vp, C.POINTER(DeviceInfo))),
    ("sync", _fn(_i, _vp)),
    ("buffer_alloc", _fn(_vp, _vp, _sz)),
    ("buffer_alloc_with_data", _fn(_vp, _vp, _vp, _sz)),
    ("buffer_free", _fn(None, _vp, _vp)),
    ("buffer_copy_to_host", _fn(_i, _vp, _vp, _vp, _sz)),
    ("buffer_copy_from_host", _fn(_i, _vp, _vp, _vp, _sz)),
    ("buffer_get_host_ptr", _fn(_vp, _vp, _vp)),
    ("kernel_load", _fn(_vp, _vp, C.c_char_p, C.c_char_p)),
    ("kernel_load_binary", _fn(_vp, _vp, _vp, _sz, C.c_char_p)),
    ("kernel_destroy", _fn(None, _vp, _vp)),
    ("kernel_dispatch", _fn(_i, _vp, _vp, _u32, _u32, _u32, _u32, _u32, _u32, C.POINTER(_vp), _i)),
    ("op_add_f32", _BIN), ("op_sub_f32", _BIN), ("op_mul_f32", _BIN), ("op_div_f32", _BIN),
    ("op_matmul_f32", _fn(_i, _vp, _vp, _vp, _vp, _i, _i, _i)),
    ("op_transpose_f32", _fn(_i, _vp, _vp, _vp, _i, _i)),
    ("op_reduce_sum_f32", _UN), ("op_reduce_max_f32", _UN), ("op_reduce_min_f32", _UN), ("op_reduce_mean_f32", _UN),
    ("op_reduce_sum_axis_f32", _fn(_i, _vp, _vp, _vp, _sz, _sz)),
    ("op_reduce_max_axis_f32", _fn(_i, _vp, _vp, _vp, _sz, _sz)),
    ("op_softmax_f32", _fn(_i, _vp, _vp, _vp, _sz, _sz)),
    ("op_log_softmax_f32", _fn(_i, _vp, _vp, _vp, _sz, _sz)),
    ("op_exp_f32", _UN), ("op_log_f32", _UN), ("op_sqrt_f32", _UN), ("op_neg_f32", _UN), ("op_abs_f32", _UN),
    ("op_tanh_f32", _UN), ("op_sigmoid_f32", _UN), ("op_relu_f32", _UN), ("op_gelu_f32", _UN),
    ("op_copy_f32", _UN),
    ("op_layer_norm_f32", _fn(_i, _vp, _vp, _vp, _vp, _vp, _sz, _sz, C.c_float)),
    ("op_rms_norm_f32", _fn(_i, _vp, _vp, _vp, _vp, _sz, _sz, C.c_float)),
    ("op_ntt_forward", _fn(_i, _vp, _vp, _sz, _u64)),
    ("op_ntt_inverse", _fn(_i, _vp, _vp, _sz, _u64)),
] + [(name, _vp) for name in (
    "op_msm", "op_poly_mul", "op_tfhe_bootstrap", "op_tfhe_keyswitch", "op_blind_rotate", "op_sample_extract",
    "op_sample_ntt", "op_poseidon2_hash", "op_blake3_hash", "op_bls12_381_add", "op_bls12_381_mul",
    "op_bls12_381_pairing", "op_bn254_add", "op_bn254_mul", "op_kzg_commit", "op_kzg_open", "op_kzg_verify",
)] + [("_reserved", _vp * 4)]


class BackendVtbl(C.Structure):
    _fields_ = _VTBL_FIELDS


class BackendDesc(C.Structure):  # backend_plugin.h:388-394
    _fields_ = [("abi_version", _u32), ("backend_name", C.c_char_p), ("backend_version", C.c_char_p),
                ("capabilities", _u32), ("vtbl", C.POINTER(BackendVtbl))]


class QmmParams(C.Structure):  # include/lux_cuda_quant.h: lux_qmm_params
    _fields_ = [(n, C.c_int32) for n in ("M", "K", "N", "bits", "group", "x_dtype", "sb_dtype", "y_dtype")]


_QMM = _fn(_i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i)


class QuantVtbl(C.Structure):  # include/lux_cuda_quant.h: lux_gpu_quant_vtbl
    _fields_ = [
        ("magic", _u32), ("version", _u32), ("size", _u32), ("_pad", _u32),
        ("qmatmul", _QMM),
        ("dequantize", _fn(_i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i)),
        ("unpack", _fn(_i, _vp, _vp, _vp, _i, _i, _i)),
        ("quantize", _fn(_i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i)),
        ("rms_norm", _fn(_i, _vp, _vp, _vp, _vp, _sz, _sz, C.c_float, _i, _i)),
        ("buffer_device_ptr", _fn(_vp, _vp, _vp)),
        ("buffer_size", _fn(_sz, _vp, _vp)),
        ("buffer_wrap", _fn(_vp, _vp, _vp, _sz)),
        ("buffer_copy_from_host_async", _fn(_i, _vp, _vp, _vp, _sz)),
        ("host_alloc_pinned", _fn(_vp, _sz)),
        ("host_free_pinned", _fn(None, _vp)),
        ("context_stream", _fn(_vp, _vp)),
        ("allocator_stats", _fn(_i, _vp, C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_u64))),
        ("allocator_trim", _fn(_i, _vp)),
        ("timer_record", _fn(_i, _vp, _i)),
        ("timer_elapsed_ms", _fn(_i, _vp, _i, _i, C.POINTER(C.c_float))),
        ("flush_l2", _fn(_i, _vp)),
        ("last_kernel", _fn(C.c_char_p, _vp)),
        ("launch_count", _fn(_u64, _vp)),
        ("graph_begin", _fn(_i, _vp)),
        ("graph_end", _fn(_i, _vp, C.POINTER(_vp))),
        ("graph_launch", _fn(_i, _vp, _vp)),
        ("graph_destroy", _fn(None, _vp)),
        ("shard_unique_id", _fn(_i, _vp)),
        ("shard_comm_create", _fn(_i, _vp, _i, _i, _vp, C.POINTER(_vp))),
        ("shard_comm_create_all", _fn(_i, C.POINTER(_vp), _i, C.POINTER(_vp))),
        ("shard_comm_destroy", _fn(None, _vp)),
        ("qmatmul_sharded", _fn(_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i)),
        ("shard_group_begin", _fn(_i)),
        ("shard_group_end", _fn(_i)),
        # version >= 2
        ("symm_alloc", _fn(_i, _vp, _i, _i, _sz, C.POINTER(_vp))),
        ("symm_export", _fn(_i, _vp, _vp)),
        ("symm_attach", _fn(_i, _vp, _vp)),
        ("symm_buffer", _fn(_vp, _vp)),
        ("symm_free", _fn(None, _vp)),
        ("qmatmul_sharded_push", _fn(_i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i)),
        # version >= 3
        ("sum3", _fn(_i, _vp, _vp, _vp, _sz, _sz, _sz)),
        ("mul_rms_norm", _fn(_i, _vp, _vp, _vp, _sz, _sz, _sz, C.c_float)),
        # version >= 4
        ("qmatmul_pro", _fn(_i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _sz, C.c_float)),
        # version >= 5
        ("qmatmul_batch", _fn(_i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i)),
        ("qmatmul_sharded_push_batch", _fn(_i, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i)),
        ("qmatmul_sharded_push_pro", _fn(_i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _sz, C.c_float)),
    ]


SYMM_HANDLE_BYTES = 96  # LUX_CUDA_SYMM_HANDLE_BYTES
PRO_RMS_NORM, PRO_SUM3 = 1, 2  # LUX_CUDA_PRO_*: prologues of qmatmul_pro


EXPORTED_SYMBOLS = ("lux_gpu_backend_init", "lux_gpu_cuda_quant_vtbl", "lux_gpu_cuda_abi_layout",
                    "lux_gpu_cuda_last_error", "lux_gpu_cuda_qmatmul_decode_noalloc")


class BackendError(RuntimeError):
    def __init__(self, code, what, detail=""):
        self.code = code
        name = ERR_NAMES[code] if 0 <= code < len(ERR_NAMES) else str(code)
        super().__init__(f"{what}: LUX_BACKEND_ERROR_{name}" + (f" ({detail})" if detail else ""))


def load_library(path=None):
    """dlopen the plugin the way the core does (RTLD_NOW | RTLD_LOCAL)."""
    path = path or os.environ.get("LUXCUDA_PLUGIN") or LIB_PATH
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path} not built: run `python -m mlx_b200.build` (needs nvcc)")
    return C.CDLL(path, mode=os.RTLD_NOW | os.RTLD_LOCAL)


class Plugin:
    """The loaded backend: descriptor, base vtable, quantized-matmul table."""

    def __init__(self, path=None, require_gpu=True):
        self.lib = load_library(path)
        self.lib.lux_gpu_backend_init.restype = C.c_bool
        self.lib.lux_gpu_backend_init.argtypes = [C.POINTER(BackendDesc)]
        self.lib.lux_gpu_cuda_quant_vtbl.restype = C.POINTER(QuantVtbl)
        self.lib.lux_gpu_cuda_last_error.restype = C.c_char_p
        self.lib.lux_gpu_cuda_qmatmul_decode_noalloc.restype = _i
        self.lib.lux_gpu_cuda_qmatmul_decode_noalloc.argtypes = [_vp] * 6 + [_i] * 6
        self.desc = BackendDesc()
        self.available = bool(self.lib.lux_gpu_backend_init(C.byref(self.desc)))
        if self.desc.abi_version != ABI_VERSION:
            raise RuntimeError(f"plugin ABI version {self.desc.abi_version}, expected {ABI_VERSION}")
        if require_gpu and not self.available:
            raise RuntimeError("libluxgpu_backend_cuda.so reports no usable B200 (lux_gpu_backend_init returned "
                               "false); this backend has no CPU fallback")
        self.vtbl = self.desc.vtbl.contents
        qp = C.cast(self.vtbl._reserved[0], C.POINTER(QuantVtbl))
        if not qp or qp.contents.magic != QUANT_MAGIC:
            raise RuntimeError("quantized-matmul extension table missing from vtbl->_reserved[0]")
        self.quant = qp.contents

    def abi_layout(self):
        out = (_u32 * 5)()
        self.lib.lux_gpu_cuda_abi_layout(out)
        return list(out)

    def last_error(self):
        return (self.lib.lux_gpu_cuda_last_error() or b"").decode()

    def device_count(self):
        n = _i(0)
        self.vtbl.get_device_count(C.byref(n))
        return n.value

    def check(self, code, what):
        if code != OK:
            raise BackendError(code, what, self.last_error())

    def context(self, device=0):
        return Context(self, device)


def _np_dtype_code(a):
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.uint16:
        return BF16
    if a.dtype == np.uint32:
        return U32
    raise TypeError(f"unsupported dtype {a.dtype}")


class Buffer:
    """A LuxBackendBuffer*; bf16 data travels as numpy uint16."""

    def __init__(self, ctx, handle, nbytes, shape=None, dtype=None, owned=True):
        self.ctx, self.handle, self.nbytes, self.shape, self.dtype, self.owned = ctx, handle, nbytes, shape, dtype, owned

    def to_host(self, shape=None, dtype=None):
        shape = self.shape if shape is None else shape
        dtype = self.dtype if dtype is None else dtype
        out = np.empty(shape, dtype=dtype)
        p = self.ctx.plugin
        p.check(p.vtbl.buffer_copy_to_host(self.ctx.handle, self.handle, out.ctypes.data_as(_vp), out.nbytes),
                "buffer_copy_to_host")
        return out

    def to_host_into(self, host_ptr, nbytes):
        """Blocking copy into caller-owned host memory (e.g. a pinned array): no allocation, no extra copy."""
        p = self.ctx.plugin
        p.check(p.vtbl.buffer_copy_to_host(self.ctx.handle, self.handle, host_ptr, nbytes), "buffer_copy_to_host")

    def from_host_ptr(self, host_ptr, nbytes):
        p = self.ctx.plugin
        p.check(p.vtbl.buffer_copy_from_host(self.ctx.handle, self.handle, host_ptr, nbytes), "buffer_copy_from_host")

    def from_host(self, a):
        a = np.ascontiguousarray(a)
        p = self.ctx.plugin
        p.check(p.vtbl.buffer_copy_from_host(self.ctx.handle, self.handle, a.ctypes.data_as(_vp), a.nbytes),
                "buffer_copy_from_host")

    @property
    def device_ptr(self):
        return self.ctx.plugin.quant.buffer_device_ptr(self.ctx.handle, self.handle)

    def free(self):
        if self.handle and not getattr(self, "borrowed", False):
            self.ctx.plugin.vtbl.buffer_free(self.ctx.handle, self.handle)
        self.handle = None


class Context:
    """A LuxBackendContext* on one GPU plus typed helpers over the two tables."""

    def __init__(self, plugin, device=0):
        self.plugin = plugin
        self.device = device
        self.handle = plugin.vtbl.create_context(device)
        if not self.handle:
            raise RuntimeError(f"create_context({device}) failed: {plugin.last_error()}")

    # --- base vtable ---------------------------------------------------------
    def close(self):
        if self.handle:
            self.plugin.vtbl.destroy_context(self.handle)
            self.handle = None

    def sync(self):
        self.plugin.check(self.plugin.vtbl.sync(self.handle), "sync")

    def device_info(self):
        info = DeviceInfo()
        self.plugin.check(self.plugin.vtbl.get_device_info(self.handle, C.byref(info)), "get_device_info")
        return info

    def alloc(self, nbytes, shape=None, dtype=None):
        h = self.plugin.vtbl.buffer_alloc(self.handle, nbytes)
        if not h:
            raise MemoryError(f"buffer_alloc({nbytes}) failed: {self.plugin.last_error()}")
        return Buffer(self, h, nbytes, shape, dtype)

    def empty(self, shape, dtype):
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        return self.alloc(n, tuple(shape), np.dtype(dtype))

    def upload(self, a):
        a = np.ascontiguousarray(a)
        h = self.plugin.vtbl.buffer_alloc_with_data(self.handle, a.ctypes.data_as(_vp), a.nbytes)
        if not h:
            raise MemoryError(f"buffer_alloc_with_data({a.nbytes}) failed: {self.plugin.last_error()}")
        return Buffer(self, h, a.nbytes, a.shape, a.dtype)

    def wrap(self, device_ptr, nbytes, shape=None, dtype=None):
        h = self.plugin.quant.buffer_wrap(self.handle, device_ptr, nbytes)
        if not h:
            raise RuntimeError("buffer_wrap failed")
        return Buffer(self, h, nbytes, shape, dtype, owned=False)

    def binary(self, op, a, b, out, n):
        self.plugin.check(getattr(self.plugin.vtbl, f"op_{op}_f32")(self.handle, a.handle, b.handle, out.handle, n),
                          f"op_{op}_f32")

    def matmul_f32(self, a, b, out, M, K, N):
        self.plugin.check(self.plugin.vtbl.op_matmul_f32(self.handle, a.handle, b.handle, out.handle, M, K, N),
                          "op_matmul_f32")

    def ntt(self, data, modulus, inverse=False):
        data = np.ascontiguousarray(data, dtype=np.uint64)
        f = self.plugin.vtbl.op_ntt_inverse if inverse else self.plugin.vtbl.op_ntt_forward
        self.plugin.check(f(self.handle, data.ctypes.data_as(_vp), data.size, modulus), "op_ntt")
        return data

    # --- quantized-matmul table ----------------------------------------------
    def qmatmul(self, x, wq, scales, biases, y, M, K, N, bits, group, x_dtype, sb_dtype, y_dtype):
        self.plugin.check(self.plugin.quant.qmatmul(self.handle, x.handle, wq.handle, scales.handle, biases.handle,
                                                    y.handle, M, K, N, bits, group, x_dtype, sb_dtype, y_dtype),
                          "qmatmul")

    def qmatmul_decode_noalloc(self, x, wq, scales, biases, y, M, K, N, bits, group, y_dtype):
        """Decode matmul through the entry point that uses the library's built-in scratch
        instead of the allocator (see include/lux_cuda_quant.h)."""
        self.plugin.check(self.plugin.lib.lux_gpu_cuda_qmatmul_decode_noalloc(
            self.handle, x.handle, wq.handle, scales.handle, biases.handle, y.handle, M, K, N, bits, group, y_dtype),
            "qmatmul_decode_noalloc")

    def qmatmul_dispatch(self, x, wq, scales, biases, y, M, K, N, bits, group, x_dtype, sb_dtype, y_dtype):
        """Same op through kernel_load / kernel_dispatch of the base vtable."""
        v = self.plugin.vtbl
        k = v.kernel_load(self.handle, None, QMM_KERNEL_NAME)
        if not k:
            raise RuntimeError("kernel_load(lux.qmm.affine) failed")
        prm = QmmParams(M, K, N, bits, group, x_dtype, sb_dtype, y_dtype)
        pb = v.buffer_alloc_with_data(self.handle, C.addressof(prm), C.sizeof(prm))
        bufs = (_vp * 6)(x.handle, wq.handle, scales.handle, biases.handle, y.handle, pb)
        try:
            self.plugin.check(v.kernel_dispatch(self.handle, k, 0, 0, 0, 0, 0, 0, bufs, 6), "kernel_dispatch")
        finally:
            v.buffer_free(self.handle, pb)
            v.kernel_destroy(self.handle, k)

    def dequantize(self, wq, scales, biases, out, N, K, bits, group, sb_dtype, out_dtype):
        self.plugin.check(self.plugin.quant.dequantize(self.handle, wq.handle, scales.handle, biases.handle,
                                                       out.handle, N, K, bits, group, sb_dtype, out_dtype),
                          "dequantize")

    def unpack(self, wq, out, N, K, bits):
        self.plugin.check(self.plugin.quant.unpack(self.handle, wq.handle, out.handle, N, K, bits), "unpack")

    def quantize(self, w, wq, scales, biases, N, K, bits, group, sb_dtype):
        self.plugin.check(self.plugin.quant.quantize(self.handle, w.handle, wq.handle, scales.handle, biases.handle,
                                                     N, K, bits, group, sb_dtype), "quantize")

    def rms_norm(self, src, dst, rows, dim, eps, in_dtype, out_dtype, weight=None):
        self.plugin.check(self.plugin.quant.rms_norm(self.handle, src.handle, dst.handle,
                                                     weight.handle if weight else None, rows, dim, eps, in_dtype,
                                                     out_dtype), "rms_norm")

    def sum3(self, src, dst, rows, cols, ld):
        """dst[r][c] = src[r][c] + src[r][cols+c] + src[r][2*cols+c] (bf16, fp32 adds)."""
        self.plugin.check(self.plugin.quant.sum3(self.handle, src.handle, dst.handle, rows, cols, ld), "sum3")

    def mul_rms_norm(self, src, dst, rows, cols, ld, eps):
        """dst = rms_norm(bf16(src[r][c] * src[r][cols+c])) per row (bf16, fp32 math)."""
        self.plugin.check(self.plugin.quant.mul_rms_norm(self.handle, src.handle, dst.handle, rows, cols, ld, eps), "mul_rms_norm")

    def qmatmul_pro(self, x, wq, scales, biases, y, M, K, N, bits, group, y_dtype, prologue, x_ld, eps=0.0):
        """y = prologue(x) . dequant(Wq)^T in one decode launch (M <= 8, bf16): PRO_RMS_NORM | PRO_SUM3."""
        self.plugin.check(self.plugin.quant.qmatmul_pro(self.handle, x.handle, wq.handle, scales.handle, biases.handle, y.handle,
                                                        M, K, N, bits, group, y_dtype, prologue, x_ld, eps), "qmatmul_pro")

    def qmatmul_batch(self, xs, wqs, scales, biases, ys, Ms, K, N, bits, group, y_dtype):
        """Independent decode matmuls of one shape (lists of buffers, one M per item) in one call."""
        n = len(xs)
        arr = lambda bufs: (C.c_void_p * n)(*[b.handle.value if isinstance(b.handle, C.c_void_p) else C.cast(b.handle, C.c_void_p).value for b in bufs])
        keep = [arr(xs), arr(wqs), arr(scales), arr(biases), arr(ys), (C.c_int * n)(*Ms)]
        self.plugin.check(self.plugin.quant.qmatmul_batch(self.handle, n, *[C.cast(a, C.c_void_p) for a in keep], K, N, bits, group, y_dtype),
                          "qmatmul_batch")

    def timer_record(self, slot):
        self.plugin.check(self.plugin.quant.timer_record(self.handle, slot), "timer_record")

    def timer_elapsed_ms(self, a, b):
        ms = C.c_float(0)
        self.plugin.check(self.plugin.quant.timer_elapsed_ms(self.handle, a, b, C.byref(ms)), "timer_elapsed_ms")
        return ms.value

    def flush_l2(self):
        self.plugin.check(self.plugin.quant.flush_l2(self.handle), "flush_l2")

    def last_kernel(self):
        return (self.plugin.quant.last_kernel(self.handle) or b"").decode()

    def launch_count(self):
        return int(self.plugin.quant.launch_count(self.handle))

    def allocator_stats(self):
        r, u, n = _u64(0), _u64(0), _u64(0)
        self.plugin.check(self.plugin.quant.allocator_stats(self.handle, C.byref(r), C.byref(u), C.byref(n)),
                          "allocator_stats")
        return {"reserved": r.value, "in_use": u.value, "driver_allocs": n.value}

    def stream(self):
        return self.plugin.quant.context_stream(self.handle)

    def graph_begin(self):
        self.plugin.check(self.plugin.quant.graph_begin(self.handle), "graph_begin")

    def graph_end(self):
        g = _vp(None)
        self.plugin.check(self.plugin.quant.graph_end(self.handle, C.byref(g)), "graph_end")
        return g

    def graph_launch(self, g):
        self.plugin.check(self.plugin.quant.graph_launch(self.handle, g), "graph_launch")

    def graph_destroy(self, g):
        self.plugin.quant.graph_destroy(g)

    def pinned_array(self, shape, dtype):
        """numpy array over page-locked host memory (host_alloc_pinned); freed with free_pinned_array."""
        dtype = np.dtype(dtype)
        nbytes = int(np.prod(shape)) * dtype.itemsize
        ptr = self.plugin.quant.host_alloc_pinned(max(nbytes, 1))
        if not ptr:
            raise MemoryError("host_alloc_pinned failed")
        buf = (C.c_char * max(nbytes, 1)).from_address(ptr)
        arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)
        self._pinned = getattr(self, "_pinned", {})
        self._pinned[arr.ctypes.data] = ptr
        return arr

    def free_pinned_array(self, arr):
        ptr = getattr(self, "_pinned", {}).pop(arr.ctypes.data, None)
        if ptr:
            self.plugin.quant.host_free_pinned(ptr)

    def upload_async(self, buf, pinned_ptr, nbytes):
        self.plugin.check(self.plugin.quant.buffer_copy_from_host_async(self.handle, buf.handle, pinned_ptr, nbytes),
                          "buffer_copy_from_host_async")


class SymmBuffer:
    """One rank's copy of y_full[M, world*N_local] that the peers store into (symm_* entry points)."""

    def __init__(self, ctx, rank, world, shape, dtype):
        self.ctx, self.rank, self.world = ctx, rank, world
        self.shape, self.dtype = tuple(shape), np.dtype(dtype)
        nbytes = int(np.prod(shape)) * self.dtype.itemsize
        h = _vp()
        ctx.plugin.check(ctx.plugin.quant.symm_alloc(ctx.handle, rank, world, nbytes, C.byref(h)), "symm_alloc")
        self.handle = h
        self.buffer = Buffer(ctx, ctx.plugin.quant.symm_buffer(h), nbytes, self.shape, self.dtype, owned=False)
        self.buffer.borrowed = True  # lives inside the symmetric buffer: never handed to buffer_free

    def export(self):
        out = (C.c_ubyte * SYMM_HANDLE_BYTES)()
        self.ctx.plugin.check(self.ctx.plugin.quant.symm_export(self.handle, out), "symm_export")
        return bytes(out)

    def attach(self, handles):
        """handles: the export() of every rank, in rank order."""
        blob = b"".join(handles)
        assert len(blob) == SYMM_HANDLE_BYTES * self.world
        buf = (C.c_ubyte * len(blob)).from_buffer_copy(blob)
        self.ctx.plugin.check(self.ctx.plugin.quant.symm_attach(self.handle, buf), "symm_attach")

    def qmatmul(self, x, wq, scales, biases, M, K, N_local, bits, group, y_dtype):
        self.ctx.plugin.check(
            self.ctx.plugin.quant.qmatmul_sharded_push(self.handle, x.handle, wq.handle, scales.handle, biases.handle,
                                                       M, K, N_local, bits, group, y_dtype), "qmatmul_sharded_push")

    def qmatmul_pro(self, x, wq, scales, biases, M, K, N_local, bits, group, y_dtype, prologue, x_ld, eps=0.0):
        """qmatmul with PRO_RMS_NORM | PRO_SUM3 applied to the (whole, gathered) x as the kernel loads it (M <= 8)."""
        self.ctx.plugin.check(
            self.ctx.plugin.quant.qmatmul_sharded_push_pro(self.handle, x.handle, wq.handle, scales.handle, biases.handle,
                                                           M, K, N_local, bits, group, y_dtype, prologue, x_ld, eps),
            "qmatmul_sharded_push_pro")

    def qmatmul_batch(self, xs, wqs, scales, biases, y_offsets, Ms, K, N_local, bits, group, y_dtype):
        """n independent matmuls of one column-sharded shape; item i's y[M_i, world*N_local] lies at byte offset
        y_offsets[i] of this buffer on every rank (qmatmul_sharded_push_batch)."""
        n = len(xs)
        assert all(len(a) == n for a in (wqs, scales, biases, y_offsets, Ms))
        keep = [(C.c_void_p * n)(*[b.handle.value if isinstance(b.handle, C.c_void_p) else C.cast(b.handle, C.c_void_p).value for b in arr])
                for arr in (xs, wqs, scales, biases)]
        offs = (C.c_size_t * n)(*[int(o) for o in y_offsets])
        ms = (C.c_int * n)(*[int(m) for m in Ms])
        self.ctx.plugin.check(
            self.ctx.plugin.quant.qmatmul_sharded_push_batch(self.handle, n, *[C.cast(a, C.c_void_p) for a in keep],
                                                             C.cast(offs, C.c_void_p), C.cast(ms, C.c_void_p),
                                                             K, N_local, bits, group, y_dtype), "qmatmul_sharded_push_batch")

    def to_host(self):
        return self.buffer.to_host(self.shape, self.dtype)

    def item_to_host(self, offset, shape, dtype):
        """The output at byte `offset` of the buffer as an array of `shape`."""
        dtype = np.dtype(dtype)
        flat = self.buffer.to_host((self.buffer.nbytes,), np.uint8)
        n = int(np.prod(shape)) * dtype.itemsize
        return flat[offset:offset + n].view(dtype).reshape(shape).copy()

    def free(self):
        if self.handle:
            self.ctx.plugin.quant.symm_free(self.handle)
            self.handle = None


class QuantizedLinear:
    """One quantized layer resident on a context: y = x . dequant(Wq)^T."""

    def __init__(self, ctx, wq, scales, biases, K, bits, group):
        self.ctx, self.K, self.bits, self.group = ctx, K, bits, group
        self.N = wq.shape[0]
        self.sb_dtype = _np_dtype_code(scales)
        self.wq, self.scales, self.biases = ctx.upload(wq), ctx.upload(scales), ctx.upload(biases)

    def __call__(self, x_buf, y_buf, M, x_dtype, y_dtype):
        self.ctx.qmatmul(x_buf, self.wq, self.scales, self.biases, y_buf, M, self.K, self.N, self.bits, self.group,
                         x_dtype, self.sb_dtype, y_dtype)

    def free(self):
        for b in (self.wq, self.scales, self.biases):
            b.free()
