"""B200-native drop-in for the `vectorlink_gpu` package: ANN graph build and beam search over
fp32 vectors, backed by hand-written sm_100a kernels in libvlgpu.so (no CPU fallback)."""
from .ann import ANN  # noqa: F401
from .queue import Queue  # noqa: F401

__all__ = ["ANN", "Queue"]
