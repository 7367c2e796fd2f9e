"""TEST INFRASTRUCTURE: ctypes wrapper around oracle/_ref/libmmamx_ref.so — the reference's own AMX kernels.

available() is False when the shared object has not been built (it is built only where the reference tree is
mounted) or the host CPU lacks AMX; callers then fall back to oracle.port.
"""
import ctypes
import os
import sys
import numpy as np
from ._common import ptr, c_contig, c_int, c_float, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "_ref", "libmmamx_ref.so")
_LIB = None

K_BF16, K_S8, K_W8 = 0, 1, 2
F32, BF16, S8 = 0, 1, 2
_NP = {F32: np.float32, BF16: np.uint16, S8: np.int8}


def cpu_has_amx():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    fl = set(line.split(":", 1)[1].split())
                    return {"amx_tile", "amx_bf16", "amx_int8", "avx512_bf16"} <= fl
    except OSError:
        pass
    return False


def available():
    return os.path.exists(_PATH) and cpu_has_amx()


def lib():
    global _LIB
    if _LIB is None:
        if not available():
            raise RuntimeError("reference AMX shim unavailable (not built, or no AMX on this CPU)")
        os.environ.setdefault("MALLOC_ARENA_MAX", "1")
        _LIB = ctypes.CDLL(_PATH)
        for name in ("ref_fc_create", "ref_mlp_create", "ref_mlp_act"):
            getattr(_LIB, name).restype = c_void_p
        # the reference prints a banner on stdout when it obtains the AMX tile permission: keep stdout clean
        sys.stdout.flush()
        saved = os.dup(1)
        devnull = os.open(os.devnull, os.O_WRONLY)
        try:
            os.dup2(devnull, 1)
            rc = _LIB.ref_init()
        finally:
            os.dup2(saved, 1); os.close(saved); os.close(devnull)
        if rc != 0:
            raise RuntimeError("AMX tile permission request failed")
    return _LIB


def max_threads():
    return lib().ref_max_threads()


class FC:
    """One reference Matmul object per thread over an N split (MatmulMTOMP, main.cpp:442-479)."""

    def __init__(self, kind, constB=True, transposeB=False, nthr=1):
        self.kind, self.transposeB, self.nthr = kind, transposeB, nthr
        self.h = c_void_p(lib().ref_fc_create(c_int(kind), c_int(int(constB)), c_int(int(transposeB)), c_int(nthr)))

    def __del__(self):
        if getattr(self, "h", None):
            lib().ref_fc_free(self.h); self.h = None

    def _dims(self, A, B):
        M, K = A.shape
        N = B.shape[0] if self.transposeB else B.shape[1]
        assert (B.shape[1] if self.transposeB else B.shape[0]) == K
        return M, K, N

    def run(self, A, B, steps=0, out_dtype=F32, bias=None, deq_scale=1.0, q_scale=1.0, q_scale_per_oc=None):
        dt = np.int8 if self.kind == K_S8 else np.uint16
        A = c_contig(A, dt); B = c_contig(B, dt)
        M, K, N = self._dims(A, B)
        f = lambda a: None if a is None else c_contig(a, np.float32)
        bias, q_scale_per_oc = f(bias), f(q_scale_per_oc)
        # the reference functor loads bias / per-channel scales in full 16-lane vectors: pad them
        pad = lambda a: None if a is None else np.concatenate([a, np.zeros(32, np.float32)])
        bias_p, qoc_p = pad(bias), pad(q_scale_per_oc)
        C = np.zeros((M, N), _NP[out_dtype])
        rc = lib().ref_fc_run(self.h, ptr(A), c_int(A.strides[0]), ptr(B), c_int(B.strides[0]), c_int(M), c_int(K),
                              c_int(N), c_int(steps), ptr(bias_p), c_float(deq_scale), c_float(q_scale), ptr(qoc_p),
                              c_int(out_dtype), ptr(C), c_int(C.strides[0]))
        assert rc == 0, rc
        return C

    def run_raw(self, A, B):
        dt = np.int8 if self.kind == K_S8 else np.uint16
        A = c_contig(A, dt); B = c_contig(B, dt)
        M, K, N = self._dims(A, B)
        C = np.zeros((M, N), np.int32 if self.kind == K_S8 else np.float32)
        rc = lib().ref_fc_run_raw(self.h, ptr(A), c_int(A.strides[0]), ptr(B), c_int(B.strides[0]), c_int(M),
                                  c_int(K), c_int(N), ptr(C), c_int(N))
        assert rc == 0, rc
        return C

    def run_w8_per_channel(self, A, B, scale, bias=None):
        A = c_contig(A, np.uint16); B = c_contig(B, np.uint16)
        M, K, N = self._dims(A, B)
        scale = c_contig(scale, np.float32)
        bias = None if bias is None else c_contig(bias, np.float32)
        C = np.zeros((M, N), np.uint16)
        rc = lib().ref_fc_run_w8_per_channel(self.h, ptr(A), c_int(A.strides[0]), ptr(B), c_int(B.strides[0]),
                                             c_int(M), c_int(K), c_int(N), ptr(scale), ptr(bias), ptr(C), c_int(N))
        assert rc == 0, rc
        return C

    def w8_scales(self):
        q, d = c_float(), c_float()
        assert lib().ref_fc_w8_scales(self.h, ctypes.byref(q), ctypes.byref(d)) == 0
        return q.value, d.value


def matvec_bf16(A, b):
    A = c_contig(A, np.uint16); b = c_contig(b, np.uint16)
    c = np.zeros(A.shape[0], np.float32)
    lib().ref_matvec_bf16(ptr(A), c_int(A.strides[0]), c_int(A.shape[0]), c_int(A.shape[1]), ptr(b), ptr(c))
    return c


def matvec_s8(A, b):
    A = c_contig(A, np.int8); b = c_contig(b, np.int8)
    c = np.zeros(A.shape[0], np.int32)
    lib().ref_matvec_s8(ptr(A), c_int(A.strides[0]), c_int(A.shape[0]), c_int(A.shape[1]), ptr(b), ptr(c))
    return c


def gemavb(A, b):
    A = c_contig(A, np.uint16); b = c_contig(b, np.uint16).copy()
    c = np.zeros(A.shape[0], np.float32)
    lib().ref_gemavb(ptr(A), c_int(A.strides[0]), c_int(A.shape[0]), c_int(A.shape[1]), ptr(b), ptr(c))
    return c


def gelu(x):
    x = c_contig(x, np.float32); assert x.size % 16 == 0
    y = np.empty_like(x); lib().ref_gelu(ptr(x), ptr(y), c_int(x.size)); return y


def silu(x):
    x = c_contig(x, np.float32); assert x.size % 16 == 0
    y = np.empty_like(x); lib().ref_silu(ptr(x), ptr(y), c_int(x.size)); return y


class MLP:
    """Fused Llama MLP arithmetic of tests/amx-mlp.cpp around the reference Matmul (see ref_harness.cpp)."""

    def __init__(self, gate, up, down, nthr=1):
        self.gate = c_contig(gate, np.uint16); self.up = c_contig(up, np.uint16)
        self.down = c_contig(down, np.uint16)
        self.N, self.K = self.gate.shape
        assert self.down.shape == (self.K, self.N)
        h = lib().ref_mlp_create(ptr(self.gate), ptr(self.up), ptr(self.down), c_int(self.K), c_int(self.N),
                                 c_int(nthr))
        assert h, "reference MLP needs N % 256 == 0 and K % 256 == 0"
        self.h = c_void_p(h)

    def __del__(self):
        if getattr(self, "h", None):
            lib().ref_mlp_free(self.h); self.h = None

    def run(self, x, want_act=False):
        x = c_contig(x, np.uint16)
        M = x.shape[0]
        out = np.zeros((M, self.K), np.uint16)
        rc = lib().ref_mlp_run(self.h, ptr(x), c_int(x.strides[0]), c_int(M), ptr(out), c_int(out.strides[0]))
        assert rc == 0
        if want_act:
            p = lib().ref_mlp_act(self.h)
            act = np.ctypeslib.as_array(ctypes.cast(p, ctypes.POINTER(ctypes.c_uint16)), shape=(M, self.N)).copy()
            return out, act
        return out
