"""B200-native (sm_100a) implementation of kernel-set's quantized-GEMM path.

``import kernel_set_b200 as ks`` gives the same module layout the reference's
``kernel_set`` package has for this path: ``ks.dispatch`` (operator layer),
``ks.gemm`` / ``ks.quant`` / ``ks.moe`` / ``ks.activation`` / ``ks.norm`` / ``ks.int4`` (out-parameter wrappers over the C
ABI), ``ks.runtime``, ``ks.KernelSetError``, ``ks.DType``.

Importing the package loads ``libkernel_set.so``; there is no CPU
implementation, so a missing library is an ``OSError`` at import.
"""
from . import _lib
from ._lib import KernelSetError, LIB_PATH
from .enums import DType, Int4Packing, Int4Source, MemcpyKind, Status
from . import _tensor, runtime, gemm, quant, moe, activation, norm, int4, dispatch  # noqa: E402
from .runtime import backend_name, device_count, version

__version__ = "0.2.1+b200"

__all__ = ["KernelSetError", "DType", "Status", "MemcpyKind", "runtime", "gemm", "quant", "moe", "activation", "norm", "int4", "dispatch",
           "Int4Source", "Int4Packing",
           "version", "backend_name", "device_count", "LIB_PATH"]
