"""B200 (sm_100a) implementation of the quantized MoE feed-forward path of the
qk inference engine: CUDA kernels behind the C ABI of include/qk_moe.h, a ctypes
binding of it, and seeded synthetic tensors for tests and benchmarks.

The directory name contains a hyphen, so the package is loaded by path (see
`__graft_entry__.package()` at the repository root) and registers itself as
`qwen_kernel_b200`.
"""
from . import synth  # noqa: F401
from .binding import (Context, DevBuf, QkmError, SEL_DTYPE, SIGNATURES, LIB_PATH,  # noqa: F401
                      load_library)
from .build import build  # noqa: F401
