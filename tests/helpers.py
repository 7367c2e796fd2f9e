"""Shared test helpers: seeded inputs, device buffers (torch is used for device memory only), C-ABI calls."""
import numpy as np

from oracle import port
from oracle._common import bf16_bits, bf16_to_f32
from mm_amx_b200 import capi

NP_OF = {capi.F32: np.float32, capi.BF16: np.uint16, capi.S8: np.int8, capi.S32: np.int32, capi.U8: np.uint8}


def two_valued_bf16(rng, shape):
    """+-0.5 like tensor2D::fill_rnd (include/tensor2D.hpp:145-172): every partial sum is exact in fp32."""
    return bf16_bits(rng.choice(np.array([-0.5, 0.5], np.float32), shape))


def two_valued_s8(rng, shape):
    return rng.choice(np.array([-1, 1], np.int8), shape)


def uniform_bf16(rng, shape, lo=-1.0, hi=1.0):
    return bf16_bits(rng.uniform(lo, hi, shape).astype(np.float32))


def normal_bf16(rng, shape, std=1.0):
    return bf16_bits((rng.standard_normal(shape) * std).astype(np.float32))


class Dev:
    """A device copy of a numpy array (raw bytes)."""

    def __init__(self, arr=None, shape=None, dtype=None, fill=None):
        import torch
        if arr is not None:
            arr = np.ascontiguousarray(arr)
            self.shape, self.dtype = arr.shape, arr.dtype
            self.t = torch.from_numpy(arr.view(np.uint8).reshape(-1).copy()).cuda()
        else:
            self.shape, self.dtype = tuple(shape), np.dtype(dtype)
            n = int(np.prod(self.shape)) * self.dtype.itemsize
            self.t = torch.zeros(max(n, 1), dtype=torch.uint8, device="cuda")
            if fill is not None:
                self.t.fill_(fill)

    @property
    def ptr(self):
        return self.t.data_ptr()

    @property
    def ld(self):
        return self.shape[-1] * self.dtype.itemsize

    def numpy(self):
        import torch
        torch.cuda.synchronize()
        n = int(np.prod(self.shape)) * self.dtype.itemsize
        return self.t[:n].cpu().numpy().view(self.dtype).reshape(self.shape).copy()


def pack(B, transposeB=False, mode=capi.PACK_PLAIN, scales=None, from_host=False):
    """B: numpy [K,N] (or [N,K] when transposeB) of uint16 (bf16 bits) / int8 / uint8."""
    dt = {np.dtype(np.uint16): capi.BF16, np.dtype(np.int8): capi.S8, np.dtype(np.uint8): capi.U8}[B.dtype]
    B = np.ascontiguousarray(B)
    K, N = (B.shape[1], B.shape[0]) if transposeB else B.shape
    sc = None
    if scales is not None:
        sc = Dev(np.ascontiguousarray(scales, np.float32))
    if from_host:
        w = capi.Weight(B.ctypes.data, dt, K, N, B.strides[0], transposeB, mode, None if sc is None else sc.ptr)
    else:
        d = Dev(B)
        w = capi.Weight(d.ptr, dt, K, N, B.strides[0], transposeB, mode, None if sc is None else sc.ptr)
    w._keep = (B, sc)
    return w


def run_matmul(w, A, out_dtype, steps=0, bias=None, deq_scale=1.0, deq_scale_per_oc=None, q_scale=1.0,
               q_scale_per_oc=None, n0=0, n1=None, sentinel=True):
    """Device-pointer C-ABI call.  Returns C [M, N_total] (columns outside [n0,n1) keep the sentinel fill)."""
    A = np.ascontiguousarray(A)
    dtA = {np.dtype(np.uint16): capi.BF16, np.dtype(np.int8): capi.S8, np.dtype(np.uint8): capi.U8}[A.dtype]
    M, K = A.shape
    N = w.N
    n1 = N if n1 is None else n1
    out_cols = N // 2 if steps & capi.STEP_SILU_MUL else N
    dA = Dev(A)
    dC = Dev(shape=(M, out_cols), dtype=NP_OF[out_dtype], fill=0xCD if sentinel else 0)
    keep = []
    def d(a):
        if a is None:
            return None
        x = Dev(np.ascontiguousarray(a, np.float32)); keep.append(x); return x.ptr
    ep = capi.make_epilogue(dC.ptr, dC.ld, out_dtype, steps, d(bias), deq_scale, d(deq_scale_per_oc), q_scale,
                            d(q_scale_per_oc))
    w.matmul(dA.ptr, dtA, M, K, A.strides[0], ep, n0, n1)
    capi.sync_check()
    return dC.numpy()


def rel_to_max(got, ref):
    """max |got - ref| / max |ref| — the tolerance measure of the bf16 paths (1e-2)."""
    got = np.asarray(got, np.float64); ref = np.asarray(ref, np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))
