"""TEST INFRASTRUCTURE: ctypes wrapper around oracle/liboracle.so (the plain C++ oracle port)."""
import ctypes
import os
import subprocess
import numpy as np
from ._common import ptr, c_contig, c_int, c_int64, c_float, c_void_p, bf16_bits, bf16_to_f32

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

DEQUANT, BIAS, GELU, QUANT = 1, 2, 4, 8
F32, BF16, S8 = 0, 1, 2
_NP = {F32: np.float32, BF16: np.uint16, S8: np.int8}


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE, "liboracle.so"])


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        _LIB = ctypes.CDLL(path)
        _LIB.orc_threads.restype = c_int
    return _LIB


def threads():
    return lib().orc_threads()


def gelu(x):
    x = c_contig(x, np.float32); y = np.empty_like(x)
    lib().orc_gelu(ptr(x), ptr(y), c_int64(x.size)); return y


def silu(x):
    x = c_contig(x, np.float32); y = np.empty_like(x)
    lib().orc_silu(ptr(x), ptr(y), c_int64(x.size)); return y


def f32_to_bf16(x):
    x = c_contig(x, np.float32); y = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16(ptr(x), ptr(y), c_int64(x.size)); return y


def gemm_bf16(A, B, transposeB=False):
    """A [M,K], B [K,N] (or [N,K] with transposeB) as bf16 bits -> fp32 accumulators [M,N]."""
    A = c_contig(A, np.uint16); B = c_contig(B, np.uint16)
    M, K = A.shape
    N = B.shape[0] if transposeB else B.shape[1]
    assert (B.shape[1] if transposeB else B.shape[0]) == K
    acc = np.empty((M, N), np.float32)
    lib().orc_gemm_bf16(ptr(A), c_int64(A.strides[0]), ptr(B), c_int64(B.strides[0]), c_int(int(transposeB)),
                        c_int(M), c_int(K), c_int(N), ptr(acc), c_int64(N))
    return acc


def gemm_i8(A, B, transposeB=False):
    """int8/uint8 A [M,K] x int8/uint8 B -> exact int32 accumulators."""
    A = np.ascontiguousarray(A); B = np.ascontiguousarray(B)
    assert A.dtype in (np.int8, np.uint8) and B.dtype in (np.int8, np.uint8)
    M, K = A.shape
    N = B.shape[0] if transposeB else B.shape[1]
    acc = np.empty((M, N), np.int32)
    lib().orc_gemm_i8(ptr(A), c_int64(A.strides[0]), c_int(int(A.dtype == np.uint8)), ptr(B), c_int64(B.strides[0]),
                      c_int(int(B.dtype == np.uint8)), c_int(int(transposeB)), c_int(M), c_int(K), c_int(N),
                      ptr(acc), c_int64(N))
    return acc


def gemm_bf16_w8(A, Wq, transposeB=False):
    A = c_contig(A, np.uint16); Wq = c_contig(Wq, np.int8)
    M, K = A.shape
    N = Wq.shape[0] if transposeB else Wq.shape[1]
    acc = np.empty((M, N), np.float32)
    lib().orc_gemm_bf16_w8(ptr(A), c_int64(A.strides[0]), ptr(Wq), c_int64(Wq.strides[0]), c_int(int(transposeB)),
                           c_int(M), c_int(K), c_int(N), ptr(acc), c_int64(N))
    return acc


def postops(acc, steps, out_dtype, bias=None, deq_scale=1.0, deq_scale_per_oc=None, q_scale=1.0,
            q_scale_per_oc=None):
    acc = np.ascontiguousarray(acc)
    assert acc.dtype in (np.float32, np.int32)
    M, N = acc.shape
    f = lambda a: None if a is None else c_contig(a, np.float32)
    bias, deq_scale_per_oc, q_scale_per_oc = f(bias), f(deq_scale_per_oc), f(q_scale_per_oc)
    C = np.empty((M, N), _NP[out_dtype])
    lib().orc_postops(ptr(acc), c_int(int(acc.dtype == np.int32)), c_int64(N), c_int(M), c_int(N), c_int(steps),
                      c_float(deq_scale), ptr(deq_scale_per_oc), ptr(bias), c_float(q_scale), ptr(q_scale_per_oc),
                      c_int(out_dtype), ptr(C), c_int64(C.strides[0]))
    return C


def quantize_weight(W):
    """bf16 bits [rows, cols] -> (int8 [rows, cols], quant_scale, dequant_scale), per-tensor absmax."""
    W = c_contig(W, np.uint16)
    Wq = np.empty(W.shape, np.int8)
    q, d = c_float(), c_float()
    lib().orc_quantize_weight(ptr(W), c_int64(W.strides[0]), c_int(W.shape[0]), c_int(W.shape[1]), ptr(Wq),
                              ctypes.byref(q), ctypes.byref(d))
    return Wq, q.value, d.value


def matvec_bf16(A, b):
    A = c_contig(A, np.uint16); b = c_contig(b, np.uint16)
    c = np.empty(A.shape[0], np.float32)
    lib().orc_matvec_bf16(ptr(A), c_int64(A.strides[0]), c_int(A.shape[0]), c_int(A.shape[1]), ptr(b), ptr(c))
    return c


def matvec_s8(A, b):
    A = c_contig(A, np.int8); b = c_contig(b, np.int8)
    c = np.empty(A.shape[0], np.int32)
    lib().orc_matvec_s8(ptr(A), c_int64(A.strides[0]), c_int(A.shape[0]), c_int(A.shape[1]), ptr(b), ptr(c))
    return c


def mlp(x, gate, up, down, want_act=False, want_partial=False):
    """x [M,K], gate/up [N,K], down [K,N] (bf16 bits) -> out [M,K] bf16 bits (+ act [M,N], + fp32 partial)."""
    x = c_contig(x, np.uint16); gate = c_contig(gate, np.uint16); up = c_contig(up, np.uint16)
    down = c_contig(down, np.uint16)
    M, K = x.shape
    N = gate.shape[0]
    assert gate.shape == (N, K) and up.shape == (N, K) and down.shape == (K, N)
    out = np.empty((M, K), np.uint16)
    act = np.empty((M, N), np.uint16) if want_act else None
    part = np.empty((M, K), np.float32) if want_partial else None
    lib().orc_mlp(ptr(x), c_int64(x.strides[0]), c_int(M), ptr(gate), ptr(up), ptr(down), c_int(K), c_int(N),
                  ptr(out), c_int64(out.strides[0]), ptr(act), ptr(part))
    res = (out,)
    if want_act:
        res += (act,)
    if want_partial:
        res += (part,)
    return res[0] if len(res) == 1 else res


def rmsnorm(x, eps, weight=None):
    """LlamaRMSNorm as the reference's benchmark script defines it (torch-ext/test.py:161-176): the row is widened to
    fp32, scaled by rsqrt(mean(x^2) + eps), rounded back to the input type (bf16).  `weight` (bf16 bits [K]) multiplies
    the rounded value and the product is rounded again (the form with a learned scale).  x: bf16 bits [M, K]."""
    xf = bf16_to_f32(np.ascontiguousarray(x, np.uint16))
    var = np.mean(xf.astype(np.float64) ** 2, axis=-1, keepdims=True).astype(np.float32)   # fp32 mean, summed exactly
    y = bf16_bits(xf * (np.float32(1.0) / np.sqrt(var + np.float32(eps))))
    if weight is not None:
        y = bf16_bits(bf16_to_f32(y) * bf16_to_f32(np.ascontiguousarray(weight, np.uint16))[None, :])
    return y


def mlp_block(x, gate, up, down, eps, norm_weight=None, add_residual=True):
    """out = (x if add_residual else 0) + MLP(RMSNorm(x)), the layer step of torch-ext/test.py:178-189 plus the residual
    of a Llama block; the sum is formed in fp32 from the MLP's fp32 result and rounded to bf16 once."""
    xn = rmsnorm(x, eps, norm_weight)
    _, part = mlp(xn, gate, up, down, want_partial=True)
    if add_residual:
        part = part + bf16_to_f32(np.ascontiguousarray(x, np.uint16))
    return bf16_bits(part)


# ---- 4-bit group-quantised weights ------------------------------------------------------------------------------------
# The reference reserves a Weight_INT4 precision (main.cpp:36) and measures only an upper bound with a dequantisation
# that does no arithmetic (fake_dequant_i4_16x32, weight_compression/wcompress.hpp:122-134); it defines no 4-bit
# algorithm.  PARITY UNPINNED: the scheme below is this library's own, the per-tensor int8 scheme of
# Matmul<bf16,int8_t,float> (include/kernels_amx.hpp:1363-1377: absmax, quant scale = range / absmax, round to
# nearest even, dequant scale = absmax / range) applied per output channel and group of 128 consecutive K.
INT4_GROUP = 128


def quantize_weight_int4(W, group=INT4_GROUP):
    """bf16 bits [N, K] -> (int8 [N, K] with values in [-7, 7], fp32 dequant scales [N, ceil(K / group)])."""
    w = bf16_to_f32(np.ascontiguousarray(W, np.uint16))
    N, K = w.shape
    G = (K + group - 1) // group
    wp = np.zeros((N, G * group), np.float32)
    wp[:, :K] = w
    wp = wp.reshape(N, G, group)
    a = np.abs(wp).max(axis=2)                                            # fp32, exact
    with np.errstate(divide="ignore"):
        qs = np.where(a > 0, np.float32(7.0) / a, np.float32(0.0)).astype(np.float32)   # fp32 division
    q = np.clip(np.rint(wp * qs[:, :, None]), -7, 7).astype(np.int8)      # fp32 product, round to nearest even
    d = (a / np.float32(7.0)).astype(np.float32)
    return q.reshape(N, G * group)[:, :K].copy(), d


def dequant_int4(q, scales, group=INT4_GROUP):
    """(int8 [N, K], fp32 [N, G]) -> fp32 [N, K]: value * scale of its group (one fp32 product)."""
    N, K = q.shape
    s = np.repeat(scales, group, axis=1)[:, :K]
    return q.astype(np.float32) * s


def gemm_bf16_w4(A, q, scales, group=INT4_GROUP):
    """bf16 bits A [M, K] x 4-bit weights (q [N, K], scales [N, G]) -> fp32 [M, N]: the integer-valued products of a
    group are summed first (exactly, float64), each group sum is scaled once, the scaled sums are added."""
    a = bf16_to_f32(np.ascontiguousarray(A, np.uint16)).astype(np.float64)
    M, K = a.shape
    N = q.shape[0]
    G = scales.shape[1]
    acc = np.zeros((M, N), np.float64)
    for j in range(G):
        k0, k1 = j * group, min(K, (j + 1) * group)
        acc += (a[:, k0:k1] @ q[:, k0:k1].astype(np.float64).T) * scales[:, j].astype(np.float64)[None, :]
    return acc.astype(np.float32)


# ---- decode attention ---------------------------------------------------------------------------------------------------
def decode_attention(q, k, v, scale=1.0, seq_lens=None):
    """One query token per sequence: q [B, H, D], k and v [B, Hkv, N, D] (bf16 bits) -> fp32 [B, H, D].
    Restates one_head_attention of the reference (include/kernels_mha.hpp:325-355: scores = q k^T, softmax over the
    keys, weighted sum of the values; the reference applies no scale, i.e. scale = 1) in float64, with query head h
    reading kv head h // (H // Hkv) and an optional per-sequence length.  Pinned: tests/golden/golden_mha_v1.npz holds
    outputs of the reference's own kernel (MHA2Kernels through oracle/ref_mha_harness.cpp) and this function agrees with
    them to 1e-6 of max |ref| (scale = 1, one kv head per query head, N a multiple of 8 — for other N the reference's
    AVX2 code itself leaves this definition); the scale, grouped heads and sequence lengths are this library's
    extensions of it."""
    qf = bf16_to_f32(np.ascontiguousarray(q, np.uint16)).astype(np.float64)
    kf = bf16_to_f32(np.ascontiguousarray(k, np.uint16)).astype(np.float64)
    vf = bf16_to_f32(np.ascontiguousarray(v, np.uint16)).astype(np.float64)
    B, H, D = qf.shape
    Hkv, N = kf.shape[1], kf.shape[2]
    G = H // Hkv
    out = np.zeros((B, H, D), np.float64)
    for b in range(B):
        n = N if seq_lens is None else int(min(max(seq_lens[b], 0), N))
        if n == 0:
            continue
        for h in range(H):
            s = scale * (kf[b, h // G, :n] @ qf[b, h])
            p = np.exp(s - s.max())
            out[b, h] = (p / p.sum()) @ vf[b, h // G, :n]
    return out.astype(np.float32)
