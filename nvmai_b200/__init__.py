"""B200-native routed-expert MoE FFN on NVMAIRepack weights: Python host bindings.

The product is `libnvmai_cuda_moe.so` (hand-written CUDA for sm_100a behind a C
ABI, `include/nvmai_cuda_moe.h`).  This package holds the build script, the
ctypes bindings the tests and the benchmark drive it through, and the blob-format
helpers.  Importing it does not load the library; the first call does, and fails
loudly when the library is absent.
"""
from . import format, synthetic  # noqa: F401
from .moe import (Elementwise, MoE, MoEConfig, NvmaiError, affine_gemv, dequant, launch_count,  # noqa: F401
                  router_noalloc)
