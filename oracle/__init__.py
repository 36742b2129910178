"""CPU oracle for the quantized-matmul path.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline
legs may import this package; the product (``mlx_b200``) never does.

PARITY UNPINNED: the reference tree has no quantized matmul and no golden
vector for one, so the packed format and the rounding rules are specified by
``qmm_oracle.c`` in this directory.  The oracle's matmul loop nest and
accumulation order are pinned against the compiled reference CPU backend
(``refcore.py``; ``src/cpu_backend.cpp:243-266``).
"""
from .oracle import *  # noqa: F401,F403
