"""TEST INFRASTRUCTURE: numpy helpers shared by the oracle wrappers (bf16 travels as uint16 bit patterns)."""
import ctypes
import numpy as np

c_void_p, c_int, c_int64, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float


def ptr(a):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


def bf16_bits(x):
    """fp32 array -> bf16 bit patterns (uint16), round to nearest even (normal values)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def c_contig(a, dtype):
    a = np.ascontiguousarray(a)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a
