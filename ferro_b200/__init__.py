"""ferro_b200: B200 (sm_100a) kernels for ferro's memory-bound device path.

`ferro_b200.backend.CudaBackend` mirrors ferro's `Backend` device methods over
the C ABI in include/ferro_b200.h (built to ferro_b200/lib/libferro_b200.so by
`python -m ferro_b200.build`).  Importing this package does not need a GPU;
constructing a backend does, and there is no CPU fallback.
"""
from . import kinds  # noqa: F401

__all__ = ["kinds"]
