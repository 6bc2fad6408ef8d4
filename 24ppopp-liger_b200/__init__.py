"""B200-native implementation of Liger's tensor-parallel transformer-layer path.

The product is the C-ABI shared library built from csrc/ (see include/liger_b200.h); this Python
package is a thin ctypes binding used by the tests and the benchmark.  PyTorch, where callers
use it, only provides device memory, streams and process-group plumbing.

There is no CPU fallback: `lib()` raises if the CUDA library has not been built, and every
compute entry point fails without a CUDA device.
"""
from . import build, capi
from .build import build_all, LIB_PATH
from .capi import lib, check, LigerError, GemmArgs, ModelConfig, default_config

__all__ = ["capi", "build_all", "LIB_PATH", "lib", "check", "LigerError", "GemmArgs", "ModelConfig", "default_config"]
