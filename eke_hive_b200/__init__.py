"""eke_hive_b200 — B200 (sm_100a) implementation of Eke Hive's quantized routed-expert path.

The compute lives in libhive_b200.so (CUDA, C ABI: include/hive_b200.h).  This package is the thin host-side mirror of
the reference engine's operator interface (hive::glm / hive::qwen free functions) over that ABI, with PyTorch used only
for device memory, streams and torch.distributed.  Importing the package loads the shared library and fails if it is
missing; nothing here computes on the CPU.
"""
from ._lib import FLAGS, HbError, load

globals().update(FLAGS)          # the HB_FLAG_* context flags of include/hive_b200.h, by name

lib = load()

from .ops import *  # noqa: E402,F401,F403
