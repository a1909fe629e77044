"""ctypes binding of the B200 tt-perf hot-path library (libb200ttperf.so, C ABI in include/b200_ttperf.h).

The directory name contains a hyphen, so load this package with `load_package()` from
`__graft_entry__` (or importlib) under the module name `ttperf_b200`.

There is no CPU fallback: importing works anywhere (so that symbol checks can run on a machine
without a GPU), but every compute call goes to the CUDA library and raises `B200Error` when the
library is missing or reports a failure.
"""
from __future__ import annotations

from . import capi, dist, nn, tensor, tp
from .tensor import DeviceTensor  # noqa: F401
from .capi import (  # noqa: F401
    ACT_GELU,
    ACT_NONE,
    ACT_RELU,
    ALGO_AUTO,
    ALGO_SIMT,
    ALGO_TCGEN05,
    BF16,
    F32,
    FP8_E4M3,
    HIFI2,
    HIFI3,
    HIFI4,
    LOFI,
    U32,
    B200Error,
    Context,
    GemmDesc,
    lib,
    lib_path,
)

__all__ = [
    "capi", "dist", "nn", "tensor", "tp", "DeviceTensor", "lib", "lib_path", "Context", "GemmDesc", "B200Error",
    "BF16", "F32", "U32", "FP8_E4M3", "ACT_NONE", "ACT_RELU", "ACT_GELU",
    "LOFI", "HIFI2", "HIFI3", "HIFI4", "ALGO_AUTO", "ALGO_TCGEN05", "ALGO_SIMT",
]
