"""GPU: decode attention (b200fc_decode_attention) against oracle.port.decode_attention (float64 restatement of
include/kernels_mha.hpp:325-355).  Bars: fp32 output within 5e-3 of max |ref| (the probabilities pass through bf16 on
their way into the tensor-core product, 2^-9 relative each), bf16 output within 1e-2."""
import os

import numpy as np
import pytest

import golden_cases as gc
import helpers as H
from mm_amx_b200 import capi
from oracle import port
from oracle._common import bf16_to_f32

pytestmark = pytest.mark.gpu


def run(q, k, v, scale, out_dtype=capi.F32, seq_lens=None, N=None):
    B, Hq, D = q.shape
    Hkv, Ncap = k.shape[1], k.shape[2]
    N = Ncap if N is None else N
    dq, dk, dv = H.Dev(q), H.Dev(k), H.Dev(v)
    out = H.Dev(shape=(B, Hq, D), dtype=H.NP_OF[out_dtype], fill=0xCD)
    es = 4 if out_dtype == capi.F32 else 2
    dl = None if seq_lens is None else H.Dev(np.asarray(seq_lens, np.int32))
    a = capi.Attention(B, Hq, Hkv, N, D, dq.ptr, Hq * D * 2, D * 2, dk.ptr, dv.ptr, Hkv * Ncap * D * 2, Ncap * D * 2, D * 2,
                       out.ptr, Hq * D * es, D * es, out_dtype, None if dl is None else dl.ptr, scale)
    capi.decode_attention(a)
    capi.sync_check()
    return out.numpy()


@pytest.mark.parametrize("B,Hq,Hkv,N,D", [
    (1, 8, 8, 17, 128), (2, 32, 32, 300, 128), (3, 64, 8, 1000, 128), (2, 16, 1, 4096, 128), (4, 8, 2, 77, 64),
    (1, 32, 4, 2049, 64), (16, 8, 8, 1, 128), (1, 4, 4, 8192, 128),
])
def test_decode_attention(B, Hq, Hkv, N, D):
    rng = np.random.default_rng(B * 7 + Hq + N + D)
    q = H.normal_bf16(rng, (B, Hq, D)); k = H.normal_bf16(rng, (B, Hkv, N, D)); v = H.normal_bf16(rng, (B, Hkv, N, D))
    scale = 1.0 / np.sqrt(D)
    ref = port.decode_attention(q, k, v, scale)
    got = run(q, k, v, scale)
    assert H.rel_to_max(got, ref) < 5e-3
    got16 = run(q, k, v, scale, capi.BF16)
    assert H.rel_to_max(bf16_to_f32(got16), ref) < 1e-2


def test_decode_attention_unscaled_like_the_reference():
    """scale = 1 (kernels_mha.hpp applies none): sharply peaked softmax, the maximum handling must hold"""
    rng = np.random.default_rng(3)
    B, Hq, Hkv, N, D = 2, 8, 8, 700, 128
    q = H.normal_bf16(rng, (B, Hq, D)); k = H.normal_bf16(rng, (B, Hkv, N, D)); v = H.normal_bf16(rng, (B, Hkv, N, D))
    ref = port.decode_attention(q, k, v, 1.0)
    assert H.rel_to_max(run(q, k, v, 1.0), ref) < 5e-3


def test_decode_attention_sequence_lengths_and_splits(monkeypatch):
    """per-sequence lengths (0, 1, ragged, full) against a cache of 1500 tokens; garbage (NaN) past each length must
    not leak; the result must not depend on how the key range is split"""
    rng = np.random.default_rng(11)
    B, Hq, Hkv, N, D = 5, 16, 4, 1500, 128
    lens = [0, 1, 37, 1024, 1500]
    q = H.normal_bf16(rng, (B, Hq, D)); k = H.normal_bf16(rng, (B, Hkv, N, D)); v = H.normal_bf16(rng, (B, Hkv, N, D))
    for b, n in enumerate(lens):
        k[b, :, n:, :] = 0x7FC0; v[b, :, n:, :] = 0x7FC0        # bf16 NaN
    scale = 1.0 / np.sqrt(D)
    ref = port.decode_attention(q, k, v, scale, lens)
    got = run(q, k, v, scale, seq_lens=lens)
    assert np.isfinite(got).all() and not got[0].any()
    assert H.rel_to_max(got, ref) < 5e-3


def test_decode_attention_repeated_calls_of_mixed_shapes():
    """calls of different shapes follow one another on a stream and share the workspace of the sub-states (it grows and
    is reused); every call must see only its own sub-states"""
    rng = np.random.default_rng(21)
    shapes = [(2, 8, 8, 3000, 128), (2, 8, 8, 3000, 128), (1, 16, 1, 4096, 128), (3, 16, 4, 1111, 64), (2, 8, 8, 3000, 128)]
    for B, Hq, Hkv, N, D in shapes:
        q = H.normal_bf16(rng, (B, Hq, D)); k = H.normal_bf16(rng, (B, Hkv, N, D)); v = H.normal_bf16(rng, (B, Hkv, N, D))
        scale = 1.0 / np.sqrt(D)
        ref = port.decode_attention(q, k, v, scale)
        for _ in range(2):
            assert H.rel_to_max(run(q, k, v, scale), ref) < 5e-3


def test_decode_attention_uniform_probabilities_exact():
    """q = 0 makes every probability 1/n: the output is the mean of v; with +-0.5 values and n a power of two all sums
    are exact, so fp32 output equals the oracle bit for bit"""
    rng = np.random.default_rng(5)
    B, Hq, Hkv, N, D = 2, 4, 2, 512, 128
    q = np.zeros((B, Hq, D), np.uint16)
    k = H.normal_bf16(rng, (B, Hkv, N, D)); v = H.two_valued_bf16(rng, (B, Hkv, N, D))
    ref = port.decode_attention(q, k, v, 1.0)
    got = run(q, k, v, 1.0)
    assert H.rel_to_max(got, ref) < 1e-6


def test_decode_attention_argument_errors():
    rng = np.random.default_rng(1)
    q = H.normal_bf16(rng, (1, 6, 128)); k = H.normal_bf16(rng, (1, 4, 32, 128))
    with pytest.raises(capi.B200FCError):       # 6 query heads over 4 kv heads
        run(q, k, k, 1.0)
    q = H.normal_bf16(rng, (1, 4, 96)); k = H.normal_bf16(rng, (1, 4, 32, 96))
    with pytest.raises(capi.B200FCError):       # head size 96
        run(q, k, k, 1.0)


def test_decode_attention_strided_cache_and_padded_heads():
    """a cache with room for more tokens than are used (token and head strides larger than the data), q and out as
    slices of wider buffers: every stride of the descriptor is honoured"""
    rng = np.random.default_rng(13)
    B, Hq, Hkv, N, D, Ncap, Dpad = 2, 8, 4, 130, 128, 256, 160
    q_full = H.normal_bf16(rng, (B, Hq, Dpad)); kc = H.normal_bf16(rng, (B, Hkv, Ncap, Dpad)); vc = H.normal_bf16(rng, (B, Hkv, Ncap, Dpad))
    dq, dk, dv = H.Dev(q_full), H.Dev(kc), H.Dev(vc)
    out = H.Dev(shape=(B, Hq, Dpad), dtype=np.float32, fill=0xCD)
    a = capi.Attention(B, Hq, Hkv, N, D, dq.ptr, Hq * Dpad * 2, Dpad * 2, dk.ptr, dv.ptr, Hkv * Ncap * Dpad * 2, Ncap * Dpad * 2,
                       Dpad * 2, out.ptr, Hq * Dpad * 4, Dpad * 4, capi.F32, None, 0.09)
    capi.decode_attention(a)
    capi.sync_check()
    got = out.numpy()
    ref = port.decode_attention(q_full[:, :, :D], kc[:, :, :N, :D], vc[:, :, :N, :D], 0.09)
    assert H.rel_to_max(got[:, :, :D], ref) < 5e-3
    assert (got[:, :, D:].view(np.uint32) == 0xCDCDCDCD).all()      # nothing written past the head size


GOLD_MHA = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_mha_v1.npz"))


@pytest.mark.parametrize("name", sorted(gc.mha_cases()))
def test_decode_attention_matches_the_reference(name):
    """the CUDA kernel against outputs recorded from the reference's own one-token attention (MHA2Kernels,
    include/kernels_mha.hpp:89-318; no scale factor, one kv head per query head): fp32 output within 5e-3 of max |ref|
    (the probabilities pass through bf16 on their way into the tensor-core product)"""
    case = gc.mha_cases()[name]
    inp = gc.mha_inputs(case)
    ref = GOLD_MHA[name]
    if case["K"] not in (64, 128):
        with pytest.raises(capi.B200FCError):
            run(inp["q"], inp["k"], inp["v"], 1.0)
        return
    got = run(inp["q"], inp["k"], inp["v"], 1.0)
    assert H.rel_to_max(got, ref) < 5e-3
