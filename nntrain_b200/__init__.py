"""B200-native compressed data-parallel gradient path.

The product is `libnntrain_grad_b200.so` (hand-written sm_100a CUDA behind a
C ABI, declared in include/nntrain_grad_abi.h).  This package is the thin
host-side mirror used by the tests and the benchmark: it loads the library
through ctypes and exposes checked wrappers named after the reference's
managed wrappers.  There is no CPU fallback: importing `nntrain_b200.lib`
without the built library raises.
"""
from .library import LibraryMissingError, NativeCudaError, load  # noqa: F401
