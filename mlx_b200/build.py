"""Build recipe of libluxgpu_backend_cuda.so (sm_100a only, in-tree).

The plugin is compiled against the reference's UNCHANGED ABI header
(include/lux/gpu/backend_plugin.h), taken where it lies in the reference tree
(``LUX_REFERENCE_INCLUDE`` or ``LUX_REFERENCE_ROOT``, else a directory ``reference`` beside this repository or
beside one of the directories above it); the header is not
copied into this repository.  On a machine without the reference tree the
prebuilt library is used as is.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(HERE, "lib", "obj")
LIB_NAME = "libluxgpu_backend_cuda.so"
LIB_PATH = os.path.join(LIB_DIR, LIB_NAME)

SOURCES = ["plugin.cu", "device_state.cu", "ops_basic.cu", "ops_tensor.cu", "quant_ops.cu", "quant_api.cu", "qmv_simt.cu",
           "qmv_mma.cu", "qmm_tc.cu", "shard.cu", "shard_push.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "--expt-relaxed-constexpr"]


def reference_root():
    """The reference tree: ``LUX_REFERENCE_ROOT``, else a directory ``reference`` beside this repository or beside
    one of the directories above it (a checkout of the repository further down still finds it)."""
    env = os.environ.get("LUX_REFERENCE_ROOT")
    if env:
        return env if os.path.isdir(env) else None
    d = os.path.realpath(ROOT)
    while True:
        parent = os.path.dirname(d)
        if parent == d:
            return None
        cand = os.path.join(parent, "reference")
        if os.path.exists(os.path.join(cand, "include", "lux", "gpu", "backend_plugin.h")):
            return cand
        d = parent


def reference_include():
    cands = [os.environ.get("LUX_REFERENCE_INCLUDE")]
    root = reference_root()
    if root:
        cands.append(os.path.join(root, "include"))
    for cand in cands:
        if cand and os.path.exists(os.path.join(cand, "lux", "gpu", "backend_plugin.h")):
            return cand
    return None


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False, ptxas_info=False):
    ref_inc = reference_include()
    if ref_inc is None:
        if os.path.exists(LIB_PATH):
            if verbose:
                print(f"reference headers not present; using prebuilt {LIB_PATH}")
            return LIB_PATH
        raise RuntimeError("cannot build the plugin: reference ABI header (lux/gpu/backend_plugin.h) not found "
                           "and no prebuilt library present")
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))] + \
              [os.path.join(ROOT, "include", "lux_cuda_quant.h"), os.path.join(ref_inc, "lux", "gpu", "backend_plugin.h")]
    objs, procs = [], []
    for src in SOURCES:
        sp = os.path.join(CSRC, src)
        op = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(op)
        if force or _newer(op, [sp] + headers):
            cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + \
                  ["-I", ref_inc, "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-c", sp, "-o", op]
            if verbose:
                print(" ".join(cmd))
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose or ptxas_info:
            sys.stdout.write(out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _newer(LIB_PATH, objs):
        cmd = ["nvcc", "-shared", "-o", LIB_PATH] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                            "-Xlinker", "--no-undefined", "-ldl"]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv))
