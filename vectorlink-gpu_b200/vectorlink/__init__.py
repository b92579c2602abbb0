"""The reference's README and main.py import `vectorlink` (README.md:20, main.py:1-8) while
its package directory is `vectorlink_gpu`; this alias makes both spellings work."""
import sys

import vectorlink_gpu
from vectorlink_gpu import ANN, Queue  # noqa: F401
from vectorlink_gpu import ann, constants, kernels, queue, utils  # noqa: F401

for _name in ("ann", "constants", "kernels", "queue", "utils", "log"):
    sys.modules[f"vectorlink.{_name}"] = sys.modules[f"vectorlink_gpu.{_name}"]
