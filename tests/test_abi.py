"""The C-ABI shared library loads without a GPU, exports every symbol that
include/*.h declares, and its descriptor / table layout match the plugin ABI
(include/lux/gpu/backend_plugin.h:82-394).  No compute calls here."""
import ctypes as C
import glob
import os
import re
import subprocess

import pytest

import mlx_b200
from mlx_b200 import plugin as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(h).read()
        names.update(re.findall(r"LUX_GPU_BACKEND_EXPORT\s+[\w\s\*]+?\b(\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    decl = declared_symbols()
    assert set(P.EXPORTED_SYMBOLS) <= decl and len(decl) >= 4
    lib = P.load_library()
    for name in decl:
        assert getattr(lib, name) is not None, name
    out = subprocess.run(["nm", "-D", "--defined-only", P.LIB_PATH], capture_output=True, text=True).stdout
    exported = {l.split()[-1] for l in out.splitlines() if " T " in l}
    assert decl <= exported
    # nothing else of ours leaks (hidden visibility): only the declared entry points are global text symbols
    assert {s for s in exported if s.startswith("lux")} == decl


def test_descriptor_and_layout():
    p = mlx_b200.Plugin(require_gpu=False)
    assert p.desc.abi_version == 2
    assert p.desc.backend_name == b"cuda"  # registry key of the core's loader (src/plugin_loader.hpp:227-230)
    assert p.desc.capabilities & 0x3 == 0x3  # TENSOR_OPS | MATMUL
    sizeof_vtbl, off_matmul, off_ntt, off_reserved, sizeof_desc = p.abi_layout()
    assert sizeof_vtbl == C.sizeof(P.BackendVtbl) == 512
    assert off_matmul == P.BackendVtbl.op_matmul_f32.offset
    assert off_ntt == P.BackendVtbl.op_ntt_forward.offset
    assert off_reserved == P.BackendVtbl._reserved.offset == 480
    assert sizeof_desc == C.sizeof(P.BackendDesc) == 40
    v = p.vtbl
    for name in ("create_context", "destroy_context", "get_device_count", "get_device_info", "sync", "buffer_alloc",
                 "buffer_alloc_with_data", "buffer_free", "buffer_copy_to_host", "buffer_copy_from_host",
                 "kernel_load", "kernel_dispatch", "op_add_f32", "op_sub_f32", "op_mul_f32", "op_matmul_f32",
                 "op_ntt_forward", "op_ntt_inverse"):
        assert C.cast(getattr(v, name), C.c_void_p).value, name
    for name in ("op_msm", "op_kzg_verify", "op_blake3_hash"):  # unsupported = NULL slot
        assert not getattr(v, name)
    assert not v._reserved[1] and not v._reserved[2] and not v._reserved[3]


def test_quant_table():
    p = mlx_b200.Plugin(require_gpu=False)
    q = p.quant
    assert q.magic == P.QUANT_MAGIC and q.version == 7 and q.size == C.sizeof(P.QuantVtbl)
    getter = p.lib.lux_gpu_cuda_quant_vtbl()
    assert C.addressof(getter.contents) == p.vtbl._reserved[0]
    for name, _ in P.QuantVtbl._fields_[4:]:
        assert C.cast(getattr(q, name), C.c_void_p).value, name


def test_python_mirror_follows_the_header_field_by_field():
    """The ctypes mirror is written by hand: its entries must be the header's, in the header's order."""
    text = open(os.path.join(ROOT, "include", "lux_cuda_quant.h")).read()
    body = text[text.index("typedef struct lux_gpu_quant_vtbl {"):text.index("} lux_gpu_quant_vtbl;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    in_header = re.findall(r"\(\*(\w+)\)\s*\(", body)
    in_mirror = [name for name, _ in P.QuantVtbl._fields_[4:]]
    assert in_header == in_mirror
    assert int(re.search(r"#define LUX_CUDA_SYMM_HANDLE_BYTES (\d+)", text).group(1)) == P.SYMM_HANDLE_BYTES


def test_null_arguments_are_errors_not_crashes():
    p = mlx_b200.Plugin(require_gpu=False)
    v, q = p.vtbl, p.quant
    assert v.sync(None) == P.ERR_INVALID
    assert v.get_device_count(None) == P.ERR_INVALID
    assert v.buffer_alloc(None, 16) is None
    assert v.buffer_copy_to_host(None, None, None, 0) == P.ERR_INVALID
    assert v.op_add_f32(None, None, None, None, 4) == P.ERR_INVALID
    assert v.op_matmul_f32(None, None, None, None, 1, 1, 1) == P.ERR_INVALID
    assert q.qmatmul(None, None, None, None, None, None, 1, 64, 1, 4, 64, 0, 0, 0) == P.ERR_INVALID
    assert q.dequantize(None, None, None, None, None, 1, 64, 4, 64, 0, 0) == P.ERR_INVALID
    assert q.symm_alloc(None, 0, 1, 64, None) == P.ERR_INVALID
    assert q.symm_export(None, None) == P.ERR_INVALID
    assert q.symm_attach(None, None) == P.ERR_INVALID
    assert q.symm_buffer(None) is None
    assert q.qmatmul_sharded_push(None, None, None, None, None, 1, 64, 16, 4, 64, 2) == P.ERR_INVALID
    assert q.qmatmul_sharded_push_batch(None, 1, None, None, None, None, None, None, 64, 16, 4, 64, 2) == P.ERR_INVALID
    assert q.qmatmul_sharded_push_pro(None, None, None, None, None, 1, 64, 16, 4, 64, 2, P.PRO_SUM3, 192, 0.0) == P.ERR_INVALID
    q.symm_free(None)
    v.buffer_free(None, None)
    v.destroy_context(None)


def test_tensor_op_slots_are_filled_and_reject_null():
    """The fp32 tensor ops the public API forwards (src/gpu_core.cpp:430-789) are all present; NULL handles are
    errors, not crashes."""
    p = mlx_b200.Plugin(require_gpu=False)
    v = p.vtbl
    un = ["op_reduce_sum_f32", "op_reduce_max_f32", "op_reduce_min_f32", "op_reduce_mean_f32", "op_exp_f32", "op_log_f32",
          "op_sqrt_f32", "op_neg_f32", "op_abs_f32", "op_tanh_f32", "op_sigmoid_f32", "op_relu_f32", "op_gelu_f32", "op_copy_f32"]
    for name in un:
        assert getattr(v, name)(None, None, None, 4) == P.ERR_INVALID, name
    assert v.op_transpose_f32(None, None, None, 2, 2) == P.ERR_INVALID
    for name in ("op_reduce_sum_axis_f32", "op_reduce_max_axis_f32", "op_softmax_f32", "op_log_softmax_f32"):
        assert getattr(v, name)(None, None, None, 2, 2) == P.ERR_INVALID, name
    assert v.op_layer_norm_f32(None, None, None, None, None, 1, 4, 1e-5) == P.ERR_INVALID
    assert v.op_rms_norm_f32(None, None, None, None, 1, 4, 1e-5) == P.ERR_INVALID
    assert p.quant.sum3(None, None, None, 1, 4, 12) == P.ERR_INVALID
    assert p.quant.mul_rms_norm(None, None, None, 1, 4, 8, 1e-6) == P.ERR_INVALID
    assert p.quant.qmatmul_pro(None, None, None, None, None, None, 1, 64, 1, 4, 64, 0, P.PRO_SUM3, 192, 0.0) == P.ERR_INVALID
    assert p.quant.qmatmul_batch(None, 1, None, None, None, None, None, None, 64, 1, 4, 64, 0) == P.ERR_INVALID


STUB_SRC = r"""
#include <stdint.h>
#include <stdbool.h>
/* layout of lux_gpu_backend_desc (include/lux/gpu/backend_plugin.h:388-394) */
typedef struct { uint32_t abi_version; const char* backend_name; const char* backend_version; uint32_t capabilities; const void* vtbl; } desc_t;
static void* slots[64];
__attribute__((visibility("default"))) bool lux_gpu_backend_init(desc_t* out) {
    out->abi_version = 3; out->backend_name = "cuda"; out->backend_version = "stub"; out->capabilities = 0; out->vtbl = slots;
    return true;
}
"""


def test_reference_loader_rejects_a_plugin_of_another_abi_version(tmp_path):
    """The reference loader checks the descriptor's ABI version (src/plugin_loader.hpp:213-223): a library named
    like this plugin that reports version 3 is closed again with a message, and the core falls back to its CPU
    backend.  (Host-side fault test: no GPU involved.)"""
    import subprocess
    import sys
    from oracle import refcore
    if not refcore.available():
        pytest.skip("compiled reference core not present")
    src = tmp_path / "stub.c"
    src.write_text(STUB_SRC)
    lib = tmp_path / "libluxgpu_backend_cuda.so"
    subprocess.run(["/usr/bin/gcc", "-shared", "-fPIC", "-o", str(lib), str(src)], check=True)
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from oracle import refcore\n"
            "r = refcore.RefCore(backend=refcore.BACKEND_CUDA)\n"
            "print('BACKEND', r.backend_name)\n"
            "import numpy as np\n"
            "print('MATMUL', r.matmul(np.array([[1,2],[3,4]], np.float32), np.array([[5,6],[7,8]], np.float32)).ravel().tolist())\n"
            "r.close()\n") % ROOT
    out = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, LUX_GPU_BACKEND_PATH=str(tmp_path)),
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    assert "has ABI version 3, expected 2" in out.stderr
    assert "BACKEND cpu" in out.stdout
    assert "MATMUL [19.0, 22.0, 43.0, 50.0]" in out.stdout


def test_kernel_registry_hook():
    """lux_kernel_registry_cuda_get (the reference's weak hook, src/kernel_loader.cpp:191-210) returns a table in
    the reference's format (include/lux/gpu/kernel_loader.h:70-90) that names every quantized-matmul variant."""
    class Embedded(C.Structure):
        _fields_ = [("name", C.c_char_p), ("entry_point", C.c_char_p), ("lang", C.c_int), ("source", C.c_char_p),
                    ("source_len", C.c_size_t), ("binary", C.c_void_p), ("binary_len", C.c_size_t)]

    class Registry(C.Structure):
        _fields_ = [("backend", C.c_char_p), ("kernels", C.POINTER(Embedded)), ("count", C.c_size_t)]

    lib = P.load_library()
    lib.lux_kernel_registry_cuda_get.restype = C.POINTER(Registry)
    reg = lib.lux_kernel_registry_cuda_get().contents
    assert reg.backend == b"cuda" and reg.count >= 7
    entries = [(reg.kernels[i].name.decode(), reg.kernels[i].entry_point.decode(), reg.kernels[i].lang) for i in range(reg.count)]
    variants = {e for n, e, _ in entries if n == "lux.qmm.affine"}
    assert {"qmv_mma<4,m8>", "qmv_mma<4,m16>", "qmv_mma<8,m8>", "qmv_mma<8,m16>", "qmm_tc<4>", "qmm_tc<8>", "qmm_tc<4,stream-k>",
            "qmm_tc<8,stream-k>", "qmm_tc<4,pairs>", "qmm_tc<8,pairs>", "qmv_mma<4,m8,rms>", "qmv_mma<4,m8,sum3>", "qmv_batch<4,m8>", "qmv_batch<4,m16>", "qmv_batch<8,m8>",
            "qmv_batch<8,m16>", "qmv_batch<4,m8,push>", "qmv_batch<4,m16,push>", "qmv_simt"} <= variants
    assert all(lang == 1 for _, _, lang in entries)  # LUX_KERNEL_LANG_CUDA


def test_no_gpu_means_unavailable_not_fallback():
    import torch
    p = mlx_b200.Plugin(require_gpu=False)
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    assert not p.available
    with pytest.raises(RuntimeError):
        mlx_b200.Plugin(require_gpu=True)


def test_product_does_not_touch_the_oracle():
    for path in glob.glob(os.path.join(ROOT, "mlx_b200", "**", "*"), recursive=True):
        if os.path.isfile(path) and path.endswith((".py", ".cu", ".h", ".cpp")):
            assert "oracle" not in open(path, errors="ignore").read().lower(), path
