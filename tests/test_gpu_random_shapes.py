"""Seeded random shapes through every kernel family against the oracle: ragged N, every group size and bit
width, K that does and does not fit the tensor-core k-blocks, M on both sides of the decode / prefill split,
small-N / large-K layers (K split over CTAs in the decode kernel)."""
import numpy as np
import pytest

from mlx_b200 import BF16
from test_gpu_parity import check, run_qmatmul

pytestmark = pytest.mark.gpu


def _cases(seed, n):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(n):
        bits = int(rng.choice([4, 8]))
        group = int(rng.choice([32, 64, 128]))
        kind = rng.integers(0, 4)
        if kind == 0:    # decode kernel: K a multiple of its k-block (256 weights at 4 bit, 128 at 8 bit)
            K = int(rng.integers(1, 24)) * (1024 // bits)
            M, N = int(rng.integers(1, 17)), int(rng.integers(1, 700))
        elif kind == 1:  # few rows of W, long K: the decode kernel splits K over CTAs
            K = int(rng.integers(16, 48)) * (1024 // bits)
            M, N = int(rng.integers(1, 17)), int(rng.integers(1, 70))
        elif kind == 2:  # prefill GEMM: K a multiple of 64
            K = int(rng.integers(1, 40)) * 64
            M, N = int(rng.integers(17, 300)), int(rng.integers(1, 400))
        else:            # whatever is left goes to the CUDA-core kernel
            K = int(rng.integers(1, 12)) * group
            M, N = int(rng.integers(1, 40)), int(rng.integers(1, 120))
        if K % group:
            K = (K // group + 1) * group
        out.append((M, K, N, bits, group))
    return out


@pytest.mark.parametrize("M,K,N,bits,group", _cases(20261125, 48))
def test_random_shape(ctx, oracle, M, K, N, bits, group):
    wq, s, b = oracle.make_layer(N, K, bits, group, oracle.BF16, config_id=7, layer=K, proj=N)
    x = oracle.make_x(M, K, oracle.BF16, config_id=7, layer=K, tag=M)
    y, kern = run_qmatmul(ctx, x, wq, s, b, bits, group, BF16)
    check(oracle, y, x, wq, s, b, bits, group, oracle.BF16)
    # the dispatch rule documented for callers
    lone_scale = (1024 // bits) == group and (N * (K // group)) % 2 == 1  # one scale per k-block and an odd total:
    if M <= 16 and K % (1024 // bits) == 0 and not lone_scale:           # the decode kernel copies scales in pairs
        assert kern.startswith("qmv_mma"), kern
    elif M <= 16 and K % (1024 // bits) == 0:
        assert kern.startswith("qmv_simt"), kern
    elif M > 16 and K % 64 == 0:
        assert kern.startswith("qmm_tc"), kern
    else:
        assert kern.startswith("qmv_simt"), kern
