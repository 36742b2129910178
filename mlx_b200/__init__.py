"""B200-native CUDA backend plugin for the Lux GPU core: affine 4/8-bit
quantized matmul behind the unchanged plugin ABI.

The product is ``lib/libluxgpu_backend_cuda.so`` (sources in ``csrc/``);
this package is the host-side mirror of the plugin interface used by the
tests and the benchmark.  There is no CPU fallback.
"""
from .plugin import (ABI_VERSION, BF16, F32, U32, BackendError, Buffer, Context, Plugin, QuantizedLinear,  # noqa: F401
                     LIB_PATH, EXPORTED_SYMBOLS)
from .shard import ShardSpec, shard_rows, gather_layout  # noqa: F401
