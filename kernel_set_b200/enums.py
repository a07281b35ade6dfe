"""Integer enums of the C ABI (``include/kernel_set/types.h``); mirrors
``bindings/python/kernel_set/enums.py`` of the reference project."""
from enum import IntEnum


class Status(IntEnum):
    SUCCESS = 0
    INVALID_ARGUMENT = 1
    UNSUPPORTED_DTYPE = 2
    UNSUPPORTED_SHAPE = 3
    CUDA = 4
    NOT_IMPLEMENTED = 5
    OUT_OF_MEMORY = 6
    ARCH_UNSUPPORTED = 7
    INTERNAL = 8


class DType(IntEnum):
    F32 = 0
    F16 = 1
    BF16 = 2
    F8E4M3 = 3
    F8E5M2 = 4
    F64 = 5
    I64 = 6
    I32 = 7
    I8 = 8
    U8 = 9
    I4 = 10


class MemcpyKind(IntEnum):
    HOST_TO_DEVICE = 0
    DEVICE_TO_HOST = 1
    DEVICE_TO_DEVICE = 2


class QuantMode(IntEnum):
    PER_TENSOR = 0
    PER_TOKEN = 1
    PER_CHANNEL = 2
    GROUPWISE = 3


class Int4Source(IntEnum):
    GPTQ = 0
    AWQ = 1


class Int4Packing(IntEnum):
    BYTES = 0   # uint8 [K/2, N]: what gemm_w4a16 reads
    WORDS = 1   # int32 [K/8, N]: what dequantize_int4 reads
