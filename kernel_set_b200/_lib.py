"""ctypes loader and prototypes for ``libkernel_set.so`` (sm_100a build).

Host-side mirror of ``bindings/python/kernel_set/_lib.py`` of the reference
project for the quantized-GEMM path: the same search order for the library
(``_lib.py:221-306``), the same ``KernelSetError`` (``:167-202``) and
``check`` (``:914-925``), and argtypes for the symbols this library exports
(reference ``:544-552`` w4a16, ``:572-581`` fp8 blockwise, ``:742-749`` group
quantizer, ``:689-695`` grouped GEMM).

There is no CPU implementation behind this module: if the shared library is
missing the import fails with instructions to build it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from typing import Optional

KS_SUCCESS = 0
KS_ERROR_INVALID_ARGUMENT = 1
KS_ERROR_UNSUPPORTED_DTYPE = 2
KS_ERROR_UNSUPPORTED_SHAPE = 3
KS_ERROR_CUDA = 4
KS_ERROR_NOT_IMPLEMENTED = 5
KS_ERROR_OUT_OF_MEMORY = 6
KS_ERROR_ARCH_UNSUPPORTED = 7
KS_ERROR_INTERNAL = 8

KS_DTYPE_F32 = 0
KS_DTYPE_F16 = 1
KS_DTYPE_BF16 = 2
KS_DTYPE_F8E4M3 = 3
KS_DTYPE_F8E5M2 = 4
KS_DTYPE_F64 = 5
KS_DTYPE_I64 = 6
KS_DTYPE_I32 = 7
KS_DTYPE_I8 = 8
KS_DTYPE_U8 = 9
KS_DTYPE_I4 = 10


class KernelSetError(RuntimeError):
    """A ``ks_*`` call returned a non-zero ``ks_status_t``.

    Attributes: ``status`` (int), ``status_name`` (``ks_status_string``),
    ``backend_message`` (``ks_last_error_string``), ``func`` (C symbol name).
    """

    def __init__(self, status: int, status_name: str, backend_message: str = "",
                 func: Optional[str] = None) -> None:
        self.status = status
        self.status_name = status_name
        self.backend_message = backend_message
        self.func = func
        head = f"{func} failed" if func else "kernel_set call failed"
        msg = f"{head} [{status_name} (={status})]"
        if backend_message:
            msg += f" : {backend_message}"
        super().__init__(msg)


_NAMES = ("libkernel_set.so", "kernel_set.so")


def _candidate_dirs() -> list[str]:
    here = os.path.dirname(os.path.abspath(__file__))
    dirs = []
    env_dir = os.environ.get("KERNEL_SET_LIB_DIR")
    if env_dir:
        dirs.append(env_dir)
    dirs += [os.path.join(here, "lib"), here, os.path.join(here, ".libs")]
    root = os.path.dirname(here)
    dirs += [os.path.join(root, "build"), os.path.join(root, "build", "lib"), os.path.join(root, "lib")]
    dirs += ["/usr/local/lib", "/usr/lib", "/opt/kernel_set/lib"]
    return dirs


def _load_library() -> ctypes.CDLL:
    tried = []
    explicit = os.environ.get("KERNEL_SET_LIB")
    if explicit:
        explicit = os.path.expanduser(explicit)
        tried.append(explicit)
        try:
            return ctypes.CDLL(explicit)
        except OSError:
            pass
    for d in _candidate_dirs():
        for name in _NAMES:
            full = os.path.join(d, name)
            if os.path.isfile(full):
                tried.append(full)
                try:
                    return ctypes.CDLL(full)
                except OSError:
                    continue
    for name in _NAMES:
        tried.append(f"<loader search path>/{name}")
        try:
            return ctypes.CDLL(name)
        except OSError:
            continue
    raise OSError(
        "Could not locate the kernel_set shared library (libkernel_set.so). Build it with "
        "`python -m kernel_set_b200.build` (needs nvcc), or set KERNEL_SET_LIB to its full path / "
        "KERNEL_SET_LIB_DIR to its directory. This package has no CPU fallback.\nSearched:\n  "
        + "\n  ".join(tried))


lib: ctypes.CDLL = _load_library()
LIB_PATH: str = getattr(lib, "_name", "")

_VP = c_void_p
_MISSING: list[str] = []


def _decl(name: str, argtypes, restype=c_int) -> None:
    try:
        fn = getattr(lib, name)
    except AttributeError:
        _MISSING.append(name)
        return
    fn.argtypes = argtypes
    fn.restype = restype


class DeviceProperties(ctypes.Structure):
    _fields_ = [
        ("name", ctypes.c_char * 256),
        ("compute_major", c_int), ("compute_minor", c_int),
        ("multiprocessor_count", c_int), ("max_threads_per_block", c_int),
        ("max_shared_memory_per_block", c_int), ("warp_size", c_int),
        ("total_global_memory", c_size_t),
        ("supports_bf16", c_int), ("supports_fp8", c_int), ("supports_tf32", c_int),
    ]


# runtime.h
_decl("ks_version", [], c_char_p)
_decl("ks_status_string", [c_int], c_char_p)
_decl("ks_dtype_size_bits", [c_int], c_int)
_decl("ks_dtype_name", [c_int], c_char_p)
_decl("ks_backend_name", [], c_char_p)
_decl("ks_device_count", [POINTER(c_int)])
_decl("ks_set_device", [c_int])
_decl("ks_get_device", [POINTER(c_int)])
_decl("ks_get_device_properties", [c_int, POINTER(DeviceProperties)])
_decl("ks_last_error_string", [], c_char_p)
_decl("ks_stream_create", [POINTER(_VP)])
_decl("ks_stream_destroy", [_VP])
_decl("ks_stream_synchronize", [_VP])
_decl("ks_malloc_device", [POINTER(_VP), c_size_t])
_decl("ks_free_device", [_VP])
_decl("ks_memcpy", [_VP, _VP, c_size_t, c_int, _VP])
_decl("ks_memset_device", [_VP, c_int, c_size_t, _VP])

# gemm.h
_W4A16 = [_VP, _VP, _VP, _VP, _VP, _VP, c_int64, c_int64, c_int64, c_int, c_int, _VP]
_decl("ks_gemm_w4a16", _W4A16)
_decl("ks_gemm_w4a16_static_scratch", _W4A16)
_FP8_BW = [_VP, _VP, _VP, POINTER(c_float), POINTER(c_float), c_int64, c_int64, c_int64,
           c_int, c_int, c_int, c_int, _VP]
_SCALED = [_VP, _VP, _VP, POINTER(c_float), POINTER(c_float)]
_decl("ks_gemm_fp8", _SCALED + [c_int64, c_int64, c_int64, c_int, c_int, c_int, c_int, _VP])
_decl("ks_gemm_w8a8", _SCALED + [_VP, c_int64, c_int64, c_int64, c_int, c_int, c_int, _VP])
_decl("ks_gemm_fp8_blockwise_colscale", [_VP, _VP, _VP, POINTER(c_float), c_int64, POINTER(c_float), c_int64, c_int64,
                                        c_int64, c_int, c_int, c_int, _VP])
_decl("ks_gemm_fp8_blockwise_scatter", [POINTER(_VP), c_int, c_int64, _VP, _VP, POINTER(c_float), POINTER(c_float),
                                       c_int64, c_int64, c_int64, c_int, c_int, c_int, _VP])
_decl("ks_sum_parts", [POINTER(_VP), c_int, _VP, c_int, c_int64, c_int64, c_int, c_int, _VP])
_decl("ks_gemm_fp8_blockwise", _FP8_BW)
_decl("ks_gemm_fp8_blockwise_nt", _FP8_BW)

# quant.h
_decl("ks_quantize_fp8_group", [_VP, POINTER(c_float), _VP, c_int64, c_int64, c_int, c_int, c_int, _VP])
_decl("ks_quantize_fp8_group_colscale", [_VP, POINTER(c_float), c_int64, _VP, c_int64, c_int64, c_int, c_int, _VP])
_decl("ks_dequantize_int4", [_VP, _VP, _VP, _VP, c_int64, c_int64, c_int, c_int, _VP])
_decl("ks_repack_int4", [_VP, _VP, _VP, c_int64, c_int64, c_int, _VP])
_decl("ks_int4_import_weight", [_VP, _VP, _VP, c_int64, c_int64, c_int, c_int, _VP])
_decl("ks_int4_import_zeros", [_VP, _VP, c_int64, c_int64, c_int, c_int, c_int, _VP])
_decl("ks_gather_columns", [_VP, _VP, _VP, c_int64, c_int64, c_int, _VP])

# moe.h
_decl("ks_moe_gate_softmax_topk", [POINTER(c_float), POINTER(c_int32), _VP, c_int64, c_int, c_int, c_int, c_int, _VP])
_decl("ks_moe_compute_permutation", [POINTER(c_int32), POINTER(c_int32), POINTER(c_int32), c_int64, c_int, c_int, _VP])
_decl("ks_moe_permute", [_VP, _VP, POINTER(c_int32), c_int64, c_int, c_int64, c_int, _VP])
_decl("ks_moe_permute_quant_fp8", [_VP, POINTER(c_float), _VP, POINTER(c_int32), c_int64, c_int, c_int64, c_int, c_int, _VP])
_decl("ks_moe_unpermute", [_VP, _VP, POINTER(c_int32), POINTER(c_float), c_int64, c_int, c_int64, c_int, _VP])
_decl("ks_moe_dispatch_plan", [POINTER(c_int32), POINTER(c_int32), POINTER(c_int32), POINTER(c_int32), POINTER(c_int32),
                              c_int, c_int, c_int, _VP])
_decl("ks_moe_permute_quant_fp8_scatter", [POINTER(_VP), POINTER(_VP), c_int, c_int64, POINTER(c_int32), POINTER(c_int32),
                                          c_int, c_int, _VP, POINTER(c_int32), c_int64, c_int, c_int64, c_int, c_int, _VP])
_decl("ks_moe_scatter_rows", [POINTER(_VP), c_int, c_int64, _VP, c_int64, POINTER(c_int32), POINTER(c_int32), c_int, c_int64,
                             c_int, _VP])
_decl("ks_moe_grouped_gemm", [_VP, _VP, _VP, POINTER(c_int32), c_int, c_int64, c_int64, c_int64, c_int, _VP])
_decl("ks_moe_grouped_gemm_fp8_blockwise",
      [_VP, _VP, _VP, POINTER(c_float), POINTER(c_float), POINTER(c_int32), c_int, c_int64, c_int64, c_int64,
       c_int, c_int, c_int, c_int, c_int, _VP])

# norm.h
_decl("ks_rms_norm", [_VP, _VP, _VP, c_int64, c_int64, c_float, c_int, _VP])
_decl("ks_rms_norm_quant_fp8", [_VP, POINTER(c_float), _VP, _VP, c_int64, c_int64, c_float, c_int, c_int, _VP])

# activation.h
_decl("ks_swiglu", [_VP, _VP, _VP, c_int64, c_int64, c_int, _VP])
_decl("ks_swiglu_packed", [_VP, _VP, c_int64, c_int64, c_int, _VP])
_decl("ks_swiglu_packed_quant_fp8", [_VP, POINTER(c_float), _VP, c_int64, c_int64, c_int, c_int, _VP])
_decl("ks_moe_grouped_gemm_fp8_blockwise_masked",
      [_VP, _VP, _VP, POINTER(c_float), POINTER(c_float), POINTER(c_int32), c_int, c_int64, c_int64, c_int64,
       c_int, c_int, c_int, c_int, c_int, _VP])


def status_string(status: int) -> str:
    raw = lib.ks_status_string(c_int(status))
    return raw.decode("utf-8", "replace") if raw else f"status {status}"


def last_error_string() -> str:
    raw = lib.ks_last_error_string()
    return raw.decode("utf-8", "replace") if raw else ""


def check(status: int, func: Optional[str] = None) -> None:
    """Raise :class:`KernelSetError` unless ``status`` is ``KS_SUCCESS``."""
    if status == KS_SUCCESS:
        return
    raise KernelSetError(status, status_string(status), last_error_string(), func)
