"""Library / device introspection; mirrors the part of
``bindings/python/kernel_set/runtime.py`` of the reference project that the
quantized-GEMM path and its benchmarks use."""
from __future__ import annotations

import ctypes

from . import _lib
from ._lib import check


def version() -> str:
    return _lib.lib.ks_version().decode()


def backend_name() -> str:
    return _lib.lib.ks_backend_name().decode()


def status_string(status: int) -> str:
    return _lib.status_string(status)


def last_error_string() -> str:
    return _lib.last_error_string()


def dtype_name(dtype: int) -> str:
    return _lib.lib.ks_dtype_name(int(dtype)).decode()


def dtype_size_bits(dtype: int) -> int:
    return int(_lib.lib.ks_dtype_size_bits(int(dtype)))


def device_count() -> int:
    n = ctypes.c_int(0)
    check(_lib.lib.ks_device_count(ctypes.byref(n)), "ks_device_count")
    return n.value


def set_device(device: int) -> None:
    check(_lib.lib.ks_set_device(int(device)), "ks_set_device")


def get_device() -> int:
    n = ctypes.c_int(0)
    check(_lib.lib.ks_get_device(ctypes.byref(n)), "ks_get_device")
    return n.value


def get_device_properties(device: int = 0) -> dict:
    p = _lib.DeviceProperties()
    check(_lib.lib.ks_get_device_properties(int(device), ctypes.byref(p)), "ks_get_device_properties")
    return {f: (getattr(p, f).decode() if f == "name" else getattr(p, f)) for f, _ in p._fields_}


def stream_synchronize(stream: int = 0) -> None:
    check(_lib.lib.ks_stream_synchronize(ctypes.c_void_p(stream)), "ks_stream_synchronize")
