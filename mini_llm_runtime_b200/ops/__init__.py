"""The kernels the parts call.

``current()`` returns the object whose methods are the kernels: by default the one ``CudaOps``
instance.  The only other implementations are stand-ins that tests install with ``use(...)`` to
exercise the host-side logic on a machine without a GPU, the way the reference's tests swap its
kernel for a Python oracle (tests/test_engine.py:82-101 there); the package never picks one by
itself.
"""

from __future__ import annotations

from contextlib import contextmanager

from .cuda_ops import AttentionBatch, CudaOps, KernelError

_default = CudaOps()
_active = _default


def current():
    return _active


@contextmanager
def use(backend):
    """Route the parts' kernel calls to ``backend`` inside the ``with`` block (tests only)."""
    global _active
    previous = _active
    _active = backend
    try:
        yield backend
    finally:
        _active = previous


__all__ = ["AttentionBatch", "CudaOps", "KernelError", "current", "use"]
