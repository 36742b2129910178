"""ctypes front end of the UNMODIFIED reference core library built from the
reference's own sources into ``oracle/_ref/libluxgpu_core.so`` (see Makefile).

Used only by tests and by the CPU-baseline legs of ``bench.py``: to pin the
oracle's accumulation order against the reference CPU backend's dense fp32
matmul (src/cpu_backend.cpp:243-266 through lux_tensor_matmul,
src/gpu_core.cpp:450-474), and to run the reference's public API against the
CUDA plugin (``LUX_GPU_BACKEND_PATH``).
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")
CORE_PATH = os.path.join(REF_DIR, "libluxgpu_core.so")
TEST_CORE_BIN = os.path.join(REF_DIR, "test_gpu_core")
TEST_KERNEL_LOADER_BIN = os.path.join(REF_DIR, "test_kernel_loader")

# include/lux/gpu.h:48-54
BACKEND_AUTO, BACKEND_CPU, BACKEND_METAL, BACKEND_CUDA = 0, 1, 2, 3
LUX_FLOAT32 = 0


def available():
    return os.path.exists(CORE_PATH)


class RefCore:
    """Thin wrapper over the reference public C API (include/lux/gpu.h:119-233)."""

    def __init__(self, backend=BACKEND_CPU, device=0):
        self.lib = C.CDLL(CORE_PATH)
        L = self.lib
        L.lux_gpu_create_with_device.restype = C.c_void_p
        L.lux_gpu_create_with_device.argtypes = [C.c_int, C.c_int]
        L.lux_gpu_destroy.argtypes = [C.c_void_p]
        L.lux_gpu_backend_name.restype = C.c_char_p
        L.lux_gpu_backend_name.argtypes = [C.c_void_p]
        L.lux_gpu_sync.argtypes = [C.c_void_p]
        L.lux_tensor_from_data.restype = C.c_void_p
        L.lux_tensor_from_data.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64), C.c_int, C.c_int]
        L.lux_tensor_destroy.argtypes = [C.c_void_p]
        L.lux_tensor_to_host.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        for name in ("lux_tensor_matmul", "lux_tensor_add", "lux_tensor_sub", "lux_tensor_mul"):
            f = getattr(L, name)
            f.restype = C.c_void_p
            f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        self.gpu = L.lux_gpu_create_with_device(backend, device)
        if not self.gpu:
            raise RuntimeError("lux_gpu_create_with_device failed")

    @property
    def backend_name(self):
        return self.lib.lux_gpu_backend_name(self.gpu).decode()

    def tensor(self, a):
        a = np.ascontiguousarray(a, dtype=np.float32)
        shape = (C.c_int64 * a.ndim)(*a.shape)
        t = self.lib.lux_tensor_from_data(self.gpu, a.ctypes.data_as(C.c_void_p), shape, a.ndim, LUX_FLOAT32)
        if not t:
            raise RuntimeError("lux_tensor_from_data failed")
        return t

    def to_host(self, t, shape):
        out = np.empty(shape, dtype=np.float32)
        rc = self.lib.lux_tensor_to_host(t, out.ctypes.data_as(C.c_void_p), out.nbytes)
        if rc:
            raise RuntimeError(f"lux_tensor_to_host rc={rc}")
        return out

    def free(self, *ts):
        for t in ts:
            self.lib.lux_tensor_destroy(t)

    def matmul_tensors(self, ta, tb):
        t = self.lib.lux_tensor_matmul(self.gpu, ta, tb)
        if not t:
            raise RuntimeError("lux_tensor_matmul failed")
        return t

    def matmul(self, a, b):
        """out[M,N] = a[M,K] . b[K,N] through lux_tensor_matmul."""
        ta, tb = self.tensor(a), self.tensor(b)
        tc = self.matmul_tensors(ta, tb)
        out = self.to_host(tc, (a.shape[0], b.shape[1]))
        self.free(ta, tb, tc)
        return out

    def binary(self, op, a, b):
        ta, tb = self.tensor(a), self.tensor(b)
        tc = getattr(self.lib, f"lux_tensor_{op}")(self.gpu, ta, tb)
        if not tc:
            raise RuntimeError(f"lux_tensor_{op} failed")
        out = self.to_host(tc, a.shape)
        self.free(ta, tb, tc)
        return out

    def close(self):
        if self.gpu:
            self.lib.lux_gpu_destroy(self.gpu)
            self.gpu = None
