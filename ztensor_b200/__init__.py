"""ztensor_b200: B200 (sm_100a) weight-quantized GEMV kernels behind ztensor's
kernel-library ABI, plus the host-side mirror of the engine entry points that
reach them.  The compute lives in libztq_sm100a.so (ztensor_b200/csrc)."""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
