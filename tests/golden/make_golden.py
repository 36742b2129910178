"""Regenerates tests/golden/*.npz.  Run in the build container, where the
reference tree is mounted and `make -C oracle` has produced oracle/_ref.

Each fixture holds seeded inputs in the packed format plus outputs computed by
the REFERENCE'S OWN CODE wherever it has any for the step:
  y_refcore  = lux_tensor_matmul(x, dequant(W)^T) through the unmodified
               reference core + CPU backend (src/gpu_core.cpp:450-474,
               src/cpu_backend.cpp:243-266), on weights dequantised by the oracle
               (the reference has no dequantiser);
and by the oracle for what the reference lacks (unpack, dequantised weights,
fp64 truth).  The GPU box has no reference tree: tests only read the .npz.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle as O  # noqa: E402
from oracle import refcore  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = [
    # name, M, K, N, bits, group, compute dtype
    ("f32_4b_g64", 3, 256, 48, 4, 64, O.F32),
    ("f32_8b_g128", 2, 256, 20, 8, 128, O.F32),
    ("bf16_4b_g64", 5, 512, 40, 4, 64, O.BF16),
    ("bf16_4b_g32", 1, 256, 33, 4, 32, O.BF16),
    ("bf16_4b_g128", 16, 256, 17, 4, 128, O.BF16),
    ("bf16_8b_g128", 2, 256, 24, 8, 128, O.BF16),
    ("bf16_8b_g64", 9, 384, 16, 8, 64, O.BF16),
]


def main():
    O.build()
    rc = refcore.RefCore()
    assert rc.backend_name == "cpu"
    for cid, (name, M, K, N, bits, group, dt) in enumerate(CASES):
        wq, s, b = O.make_layer(N, K, bits, group, dt, config_id=100 + cid, bias_noise=1e-3 if dt == O.F32 else 0.0)
        x = O.make_x(M, K, dt, config_id=100 + cid)
        q = O.unpack(wq, K, bits)
        w = O.dequantize(wq, s, b, K, bits, group, dt)
        wf = w if dt == O.F32 else O.from_bf16(w)
        xf = x if dt == O.F32 else O.from_bf16(x)
        y_refcore = rc.matmul(xf, np.ascontiguousarray(wf.T))
        y_oracle = O.qmatmul_ref(x, wq, s, b, bits, group, y_dtype=O.F32)
        assert np.array_equal(y_refcore, y_oracle), name
        truth = O.qmatmul_truth(x, wq, s, b, bits, group)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), M=M, K=K, N=N, bits=bits, group=group, dtype=dt,
                            x=x, wq=wq, scales=s, biases=b, q=q, w=w, y_refcore=y_refcore, truth=truth)
        print(name, "ok", O.rel_err(y_refcore, truth))
    # hand-computable known-answer words
    np.savez_compressed(os.path.join(HERE, "kat_words.npz"),
                        w4=np.array([[0x76543210, 0xFEDCBA98, 0x00000000, 0xFFFFFFFF]], dtype=np.uint32),
                        q4=np.array([list(range(16)) + [0] * 8 + [15] * 8], dtype=np.uint8),
                        w8=np.array([[0x03020100, 0xFFFE8180]], dtype=np.uint32),
                        q8=np.array([[0, 1, 2, 3, 0x80, 0x81, 0xFE, 0xFF]], dtype=np.uint8))
    rc.close()


if __name__ == "__main__":
    main()
