"""nova_compiler_b200 — B200 (sm_100a) execution backend for the Nova compiler's matmul hot path.

`ops` mirrors the nova / linalg operator surface on torch CUDA tensors; `_lib` is the ctypes view of
the C ABI (include/nova_b200.h, built into libnova_b200.so by `python -m nova_compiler_b200.build`).
"""
from . import _lib  # noqa: F401
from . import ops  # noqa: F401
from ._lib import NovaB200Error  # noqa: F401

__all__ = ["ops", "NovaB200Error"]
