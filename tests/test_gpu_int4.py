"""GPU: 4-bit group-quantised weights (B200FC_PACK_INT4_GROUP) through the C ABI, against oracle.port.

The reference reserves the precision (Weight_INT4, main.cpp:36) and measures an upper bound without arithmetic
(weight_compression/wcompress.hpp:122-134); it has no 4-bit algorithm and so no golden vectors — the oracle restates
this library's own definition (per group of 128 K: q = rne(w * (7 / absmax)), value = q * (absmax / 7)).
Bars: the stored integers and scales bit-exact; decode results (group sums exact, one fp32 scale per group) within
1e-5 of max |ref| in fp32 and 1e-2 after bf16 rounding; M > 16 (values rounded to bf16 before the GEMM) within 1e-2.
"""
import ctypes

import numpy as np
import pytest

import helpers as H
from mm_amx_b200 import capi
from oracle import port
from oracle._common import bf16_to_f32

pytestmark = pytest.mark.gpu


def stored(w):
    """(int8 [N, K], fp32 [N, groups]) as the library holds them"""
    unp = H.Dev(shape=(w.N, w.K), dtype=np.int8, fill=0x55)
    w.unpack(unp.ptr, w.K)
    groups = (w.K + capi.INT4_GROUP - 1) // capi.INT4_GROUP
    sc = np.full((w.N, groups), np.nan, np.float32)
    w.group_scales(sc.ctypes.data, sc.strides[0])
    return unp.numpy(), sc


@pytest.mark.parametrize("K,N,transposeB", [(256, 320, False), (1000, 77, True), (4096, 512, True), (384, 130, False)])
def test_int4_quantiser_bit_exact(K, N, transposeB):
    rng = np.random.default_rng(K * 3 + N)
    B = H.normal_bf16(rng, (N, K) if transposeB else (K, N), 0.02)
    if not transposeB:
        B[0:128, 5] = 0                       # an all-zero group (K 0..127 of output channel 5)
    Wnk = B if transposeB else np.ascontiguousarray(B.T)
    q, d = port.quantize_weight_int4(Wnk)
    w = H.pack(B, transposeB, capi.PACK_INT4_GROUP)
    info = w.info()
    assert info["compressed"] and info["dtype"] == capi.S4 and info["K"] == K and info["N"] == N
    got_q, got_d = stored(w)
    assert len(np.unique(q)) == 15
    assert np.array_equal(got_q, q)
    assert np.array_equal(got_d.view(np.uint32), d.view(np.uint32))


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("K,N", [(1536, 512), (1000, 1000), (4096, 4096), (256, 128), (11008, 1024)])
def test_int4_decode(M, K, N):
    rng = np.random.default_rng(M * 131 + K + N)
    x = H.normal_bf16(rng, (M, K))
    W = H.normal_bf16(rng, (N, K), 0.02)
    q, d = port.quantize_weight_int4(W)
    acc = port.gemm_bf16_w4(x, q, d)
    w = H.pack(W, True, capi.PACK_INT4_GROUP)
    got = H.run_matmul(w, x, capi.F32, steps=capi.STEP_DEQUANT)
    assert H.rel_to_max(got, acc) < 1e-5
    bias = rng.standard_normal(N).astype(np.float32)
    got16 = H.run_matmul(w, x, capi.BF16, steps=capi.STEP_DEQUANT | capi.STEP_BIAS | capi.STEP_GELU, bias=bias)
    ref16 = port.postops(acc, port.DEQUANT | port.BIAS | port.GELU, port.BF16, bias=bias)
    assert H.rel_to_max(bf16_to_f32(got16), bf16_to_f32(ref16)) < 1e-2


def test_int4_decode_exact_on_power_of_two_groups():
    """weights in {-7..7} * 2^-6 per group quantise to themselves with scale 2^-6; with +-0.5 activations every partial sum
    is exact in fp32, so the decode result must equal the oracle bit for bit whatever the order of summation"""
    rng = np.random.default_rng(9)
    M, K, N = 16, 2048, 640
    q0 = rng.integers(-7, 8, (N, K)).astype(np.float32)
    q0[:, ::128] = 7                                        # every group reaches the full range
    W = H.bf16_bits(q0 * np.float32(2.0 ** -6))
    x = H.two_valued_bf16(rng, (M, K))
    q, d = port.quantize_weight_int4(W)
    assert np.array_equal(q, q0.astype(np.int8)) and np.all(d == np.float32(2.0 ** -6))
    w = H.pack(W, True, capi.PACK_INT4_GROUP)
    for rows in (1, 5, 16):
        got = H.run_matmul(w, x[:rows], capi.F32, steps=capi.STEP_DEQUANT)
        assert np.array_equal(got, port.gemm_bf16_w4(x[:rows], q, d))


def test_int4_column_range_and_bad_n0():
    rng = np.random.default_rng(2)
    M, K, N = 4, 768, 700
    x = H.normal_bf16(rng, (M, K)); W = H.normal_bf16(rng, (N, K), 0.02)
    q, d = port.quantize_weight_int4(W)
    acc = port.gemm_bf16_w4(x, q, d)
    w = H.pack(W, True, capi.PACK_INT4_GROUP)
    for n0, n1 in [(128, 700), (256, 300), (0, 129)]:
        got = H.run_matmul(w, x, capi.F32, steps=capi.STEP_DEQUANT, n0=n0, n1=n1)
        assert H.rel_to_max(got[:, n0:n1], acc[:, n0:n1]) < 1e-5
        rest = np.delete(got, np.s_[n0:n1], axis=1).view(np.uint32)
        assert (rest == 0xCDCDCDCD).all()
    with pytest.raises(capi.B200FCError):
        H.run_matmul(w, x, capi.F32, steps=capi.STEP_DEQUANT, n0=64, n1=700)
    with pytest.raises(capi.B200FCError):           # compressed weights need STEP_DEQUANT
        H.run_matmul(w, x, capi.F32)


@pytest.mark.parametrize("M,K,N", [(40, 512, 1024), (130, 8192, 2600)])
def test_int4_prefill_blocks(M, K, N):
    """M > 16: blocks of weight rows are widened to bf16 (value * group scale, rounded) and multiplied by the GEMM"""
    rng = np.random.default_rng(M + K)
    x = H.normal_bf16(rng, (M, K)); W = H.normal_bf16(rng, (N, K), 0.02)
    q, d = port.quantize_weight_int4(W)
    bias = rng.standard_normal(N).astype(np.float32)
    w = H.pack(W, True, capi.PACK_INT4_GROUP)
    got = H.run_matmul(w, x, capi.F32, steps=capi.STEP_DEQUANT | capi.STEP_BIAS, bias=bias)
    ref = port.gemm_bf16_w4(x, q, d) + bias[None, :]
    assert H.rel_to_max(got, ref) < 1e-2
    # against the same rounding the path applies (dequantised values rounded to bf16), the GEMM is fp32-accurate
    wide = H.bf16_bits(port.dequant_int4(q, d))
    ref2 = port.gemm_bf16(x, wide, transposeB=True) + bias[None, :]
    assert H.rel_to_max(got, ref2) < 1e-5


def test_int4_export_import_round_trip(tmp_path):
    rng = np.random.default_rng(3)
    M, K, N = 40, 700, 333
    x = H.normal_bf16(rng, (M, K)); W = H.normal_bf16(rng, (K, N), 0.02)
    w = H.pack(W, False, capi.PACK_INT4_GROUP)
    blob = w.export()
    (tmp_path / "w4.bin").write_bytes(blob)
    w2 = capi.Weight.from_blob((tmp_path / "w4.bin").read_bytes())
    assert w2.info() == w.info()
    a, b = stored(w), stored(w2)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    for rows in (3, M):
        want = H.run_matmul(w, x[:rows], capi.F32, steps=capi.STEP_DEQUANT)
        got = H.run_matmul(w2, x[:rows], capi.F32, steps=capi.STEP_DEQUANT)
        assert np.array_equal(got, want)
    assert w2.export() == blob
    with pytest.raises(capi.B200FCError):
        capi.Weight.from_blob(blob[: len(blob) - 16])


def test_int4_host_buffers_and_k_major_source():
    """b200fc_matmul_host with 4-bit weights packed from a [K, N] host matrix whose K is no multiple of the group size;
    bias and GeLU behind the dequantisation, bf16 out"""
    rng = np.random.default_rng(8)
    M, K, N = 7, 1000, 384
    x = H.normal_bf16(rng, (M, K)); W = H.normal_bf16(rng, (K, N), 0.05)
    q, d = port.quantize_weight_int4(np.ascontiguousarray(W.T))
    bias = rng.standard_normal(N).astype(np.float32)
    w = H.pack(W, False, capi.PACK_INT4_GROUP, from_host=True)
    out = np.full((M, N), 0xCDCD, np.uint16)
    ep = capi.make_epilogue(out.ctypes.data, N * 2, capi.BF16, capi.STEP_DEQUANT | capi.STEP_BIAS | capi.STEP_GELU, bias.ctypes.data)
    w.matmul_host(x.ctypes.data, capi.BF16, M, K, K * 2, ep)
    ref = port.postops(port.gemm_bf16_w4(x, q, d), port.DEQUANT | port.BIAS | port.GELU, port.BF16, bias=bias)
    assert H.rel_to_max(bf16_to_f32(out), bf16_to_f32(ref)) < 1e-2


def test_int4_outliers_and_tiny_groups():
    """a group dominated by one outlier quantises the rest to zero; a group of tiny values keeps its resolution through
    its own scale — the per-group scheme's reason to exist.  Stored integers and scales still equal the oracle's."""
    rng = np.random.default_rng(4)
    N, K = 256, 512
    Wf = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    Wf[:, 5] = 3.0                       # outlier in group 0 of every row
    Wf[:, 128:256] *= 1e-4               # a tiny group
    W = H.bf16_bits(Wf)
    q, d = port.quantize_weight_int4(W)
    w = H.pack(W, True, capi.PACK_INT4_GROUP)
    unp = H.Dev(shape=(N, K), dtype=np.int8)
    w.unpack(unp.ptr, K)
    sc = np.zeros((N, 4), np.float32)
    w.group_scales(sc.ctypes.data, sc.strides[0])
    assert np.array_equal(unp.numpy(), q) and np.array_equal(sc, d)
    assert np.abs(q[:, 128:256]).max() == 7 and d[:, 1].max() < 1e-4
    x = H.normal_bf16(rng, (3, K))
    got = H.run_matmul(w, x, capi.F32, steps=capi.STEP_DEQUANT)
    assert H.rel_to_max(got, port.gemm_bf16_w4(x, q, d)) < 1e-5
