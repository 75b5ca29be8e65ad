"""kraken_b200 -- a B200 (sm_100a) backend for Kraken's quantized-weight matmul path.

The product is the C-ABI library ``libkrk_cuda.so`` (``include/krk_cuda.h``) and the
``CudaBackend`` host class (``include/krk_cuda_backend.hpp``). This package holds their
sources (``csrc/``), the in-tree build (``build.py``), a ctypes binding (``capi``), the
seeded input generator (``synth``) and the multi-GPU sharding helpers (``shard``).

``import kraken_b200`` is cheap and never touches the GPU; ``kraken_b200.capi`` loads the
library and raises if it has not been built.
"""

__all__ = ["synth", "build", "capi", "shard"]
