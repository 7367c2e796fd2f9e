"""CPU: pins the plain C++ oracle port against outputs recorded from the reference's own AMX kernels
(tests/golden/golden_v1.npz, written by tests/golden/make_golden.py).

Bit-exact where the arithmetic is exact (two-valued inputs, all integer paths, bf16->int8 weight quantisation);
otherwise the port's sequential fp32 accumulation and the AMX unit's internal summation differ in the last bits:
measured <= 2e-6 of max|ref|, asserted at 1e-5.  SiLU: the port divides exactly where the reference uses a 14-bit
reciprocal, asserted at 2^-13 relative.
"""
import os

import numpy as np
import pytest

from oracle import port
from oracle._common import bf16_bits, bf16_to_f32
import golden_cases as gc
import helpers as H

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_v1.npz"))


def gold(name):
    if name in GOLD.files:
        return GOLD[name]
    base = name[:-2]
    assert name[-2:] in ("/N", "/T") and base in GOLD.files, name
    return GOLD[base]


def port_fc(case, inp):
    tr = case["transposeB"]
    B = np.ascontiguousarray(inp["B"].T) if tr else inp["B"]
    if case["kind"] == "s8":
        acc = port.gemm_i8(inp["A"], B, tr)
    elif case["kind"] == "bf16":
        acc = port.gemm_bf16(inp["A"], B, tr)
    else:
        Wq, q, d = port.quantize_weight(inp["B"])
        acc = port.gemm_bf16_w8(inp["A"], np.ascontiguousarray(Wq.T) if tr else Wq, tr)
        if case.get("per_channel"):
            assert np.array_equal(Wq, inp["Wq"])
            return port.postops(acc, port.DEQUANT, port.BF16, deq_scale=d, deq_scale_per_oc=inp["scale"]), (q, d)
        return port.postops(acc, case["steps"], case["out"], deq_scale=d), (q, d)
    if case.get("raw"):
        return acc, None
    return port.postops(acc, case["steps"], case["out"], bias=inp.get("bias"), deq_scale=case.get("deq", 1.0),
                        q_scale=case.get("q", 1.0), q_scale_per_oc=inp.get("q_oc")), None


def compare(name, case, got, ref):
    exact = case["data"] in ("two",) or (case["kind"] == "s8" and case.get("raw"))
    if exact:
        assert np.array_equal(got, ref), name
    elif got.dtype == np.int8:
        d = np.abs(got.astype(np.int32) - ref.astype(np.int32))
        assert d.max() <= 1 and (d != 0).mean() < 2e-3, (name, d.max(), (d != 0).mean())
    elif got.dtype == np.uint16:
        g, r = bf16_to_f32(got), bf16_to_f32(ref)
        assert np.abs(g - r).max() <= np.abs(r).max() * 2.0 ** -8, name   # at most one bf16 ulp at the top
        if not (case.get("steps", 0) & gc.GELU):   # GeLU of x near -5 cancels to ~0: tiny absolute, large relative
            assert (got != ref).mean() < 2e-3, name
    else:
        assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max(), name


@pytest.mark.parametrize("name", sorted(gc.fc_cases()))
def test_fc_port_matches_reference(name):
    case = gc.fc_cases()[name]
    got, scales = port_fc(case, gc.fc_inputs(case))
    compare(name, case, got, gold(name))
    if scales is not None and not case.get("per_channel"):
        key = name + "/scales" if name + "/scales" in GOLD.files else name[:-2] + "/scales"
        assert np.array_equal(np.array(scales, np.float32), GOLD[key])


@pytest.mark.parametrize("name", sorted(gc.matvec_cases()))
def test_matvec_port_matches_reference(name):
    case = gc.matvec_cases()[name]
    inp = gc.matvec_inputs(case)
    got = port.matvec_bf16(inp["A"], inp["b"]) if case["kind"] == "bf16" else port.matvec_s8(inp["A"], inp["b"])
    assert np.array_equal(got, GOLD[name])
    if name + "/gemavb" in GOLD.files:
        assert np.array_equal(got, GOLD[name + "/gemavb"])


@pytest.mark.parametrize("name", sorted(gc.mlp_cases()))
def test_mlp_port_matches_reference(name):
    case = gc.mlp_cases()[name]
    inp = gc.mlp_inputs(case)
    out, act = port.mlp(inp["x"], inp["gate"], inp["up"], inp["down"], want_act=True)
    ra, ro = bf16_to_f32(GOLD[name + "/act"]), bf16_to_f32(GOLD[name])
    a, o = bf16_to_f32(act), bf16_to_f32(out)
    assert np.abs(a - ra).max() <= np.abs(ra).max() * 2.0 ** -8
    assert (act != GOLD[name + "/act"]).mean() < 0.02      # rcp14 vs exact division flips few bf16 roundings
    assert np.abs(o - ro).max() <= 1e-2 * np.abs(ro).max()


def test_gelu_port_matches_reference():
    x = gc.activation_points()
    got, ref = port.gelu(x), GOLD["gelu"]
    assert np.array_equal(got, ref)


def test_silu_port_close_to_reference():
    x = gc.activation_points()
    got, ref = port.silu(x), GOLD["silu"]
    ok = np.isfinite(ref)
    assert np.array_equal(np.isfinite(got), ok)
    err = np.abs(got[ok] - ref[ok])
    assert (err <= np.abs(ref[ok]) * 2.0 ** -13 + 1e-37).all()


def test_rmsnorm_oracle_matches_the_reference_script_definition():
    """port.rmsnorm against the LlamaRMSNorm of the reference's benchmark script (torch-ext/test.py:161-176), evaluated
    with torch on the CPU: identical up to the last bf16 bit (torch.mean sums in fp32, the oracle exactly)."""
    import torch
    rng = np.random.default_rng(11)
    x = (rng.standard_normal((7, 384)) * 2.0).astype(np.float32)
    xb = bf16_bits(x)
    t = torch.from_numpy(bf16_to_f32(xb)).to(torch.bfloat16)
    h = t.to(torch.float32)
    var = h.pow(2).mean(-1, keepdim=True)
    want = (h * torch.rsqrt(var + 1e-6)).to(torch.bfloat16)
    want_bits = want.view(torch.int16).numpy().view(np.uint16)
    got = port.rmsnorm(xb, 1e-6)
    assert np.abs(got.astype(np.int32) - want_bits.astype(np.int32)).max() <= 1
    assert (got == want_bits).mean() > 0.99


def test_int4_group_quantiser_properties():
    """The 4-bit scheme has no reference counterpart (parity unpinned); pin the restatement to its definition:
    group absmax maps to +-7, every value is within half a step of the original, zero groups stay zero."""
    rng = np.random.default_rng(44)
    N, K = 24, 300                                   # last group ragged (300 = 2 * 128 + 44)
    W = H.normal_bf16(rng, (N, K), std=0.02)
    W[3, 128:256] = 0                                # an all-zero group
    q, d = port.quantize_weight_int4(W)
    w = bf16_to_f32(W)
    assert q.shape == (N, K) and q.dtype == np.int8 and d.shape == (N, 3) and d.dtype == np.float32
    assert q.min() >= -7 and q.max() <= 7
    assert d[3, 1] == 0 and not q[3, 128:256].any()
    for j, (k0, k1) in enumerate([(0, 128), (128, 256), (256, 300)]):
        a = np.abs(w[:, k0:k1]).max(axis=1)
        assert np.array_equal(d[:, j], a / np.float32(7))
        hit = np.abs(q[:, k0:k1]).max(axis=1)
        assert np.all(hit[a > 0] == 7)
        err = np.abs(port.dequant_int4(q, d)[:, k0:k1] - w[:, k0:k1])
        assert np.all(err <= 0.5 * d[:, j][:, None] * (1 + 1e-6))
    # the product: per-group integer sums scaled once == a plain product with the dequantised matrix (fp64 both)
    x = H.normal_bf16(rng, (5, K))
    ref = bf16_to_f32(x).astype(np.float64) @ port.dequant_int4(q, d).astype(np.float64).T
    got = port.gemm_bf16_w4(x, q, d)
    assert np.allclose(got, ref, rtol=1e-5, atol=1e-6)


GOLD_MHA = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_mha_v1.npz"))


@pytest.mark.parametrize("name", sorted(gc.mha_cases()))
def test_decode_attention_oracle_pinned_to_the_reference(name):
    """oracle.port.decode_attention (float64, scale = 1 as in the reference) against outputs recorded from the
    reference's own one-token attention, MHA2Kernels (include/kernels_mha.hpp:89-318; fp32 AVX2, exponentials by
    polynomial, sub-states of bn tokens combined afterwards): measured <= 1e-6 of max |ref|, asserted at 1e-5."""
    case = gc.mha_cases()[name]
    inp = gc.mha_inputs(case)
    ref = GOLD_MHA[name]
    got = port.decode_attention(inp["q"], inp["k"], inp["v"], 1.0)
    assert got.shape == ref.shape
    assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max()
