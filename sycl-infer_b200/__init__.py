"""b200q: B200-native quantized GEMV/GEMM over raw GGUF blocks.

The product is the C-ABI shared library ``libb200q.so`` (CUDA, sm_100a) declared in
``include/b200q.h``.  This package holds its sources (``csrc/``), the in-tree build, a
ctypes binding and a host-side mirror of the reference engine's backend-operator
interface for this path.  The directory name carries a hyphen, so it is imported
through ``__graft_entry__.load_package()`` under the module name ``sycl_infer_b200``.
"""
from . import synth  # noqa: F401
from .capi import Lib, B200QError, load_lib  # noqa: F401
from .backend import cuda_backend, make_cuda_backend  # noqa: F401
