"""GPU: the CUDA path against outputs recorded from the reference's own AMX kernels (tests/golden/golden_v1.npz)."""
import os

import numpy as np
import pytest

from oracle._common import bf16_to_f32
from mm_amx_b200 import capi
import golden_cases as gc
import helpers as H

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_v1.npz"))
OUT = {gc.F32: capi.F32, gc.BF16: capi.BF16, gc.S8: capi.S8}


def gold(name):
    return GOLD[name] if name in GOLD.files else GOLD[name[:-2]]


@pytest.mark.parametrize("name", sorted(gc.fc_cases()))
def test_fc_matches_reference(name):
    case = gc.fc_cases()[name]
    inp = gc.fc_inputs(case)
    tr = case["transposeB"]
    ref = gold(name)
    if case["kind"] == "w8" and case.get("per_channel"):
        w = H.pack(np.ascontiguousarray(inp["Wq"].T) if tr else inp["Wq"], tr, capi.PACK_INT8_CHANNEL, inp["scale"])
        got = H.run_matmul(w, inp["A"], capi.BF16, steps=capi.STEP_DEQUANT)
    elif case["kind"] == "w8":
        w = H.pack(np.ascontiguousarray(inp["B"].T) if tr else inp["B"], tr, capi.PACK_QUANT_TENSOR)
        key = name + "/scales" if name + "/scales" in GOLD.files else name[:-2] + "/scales"
        assert np.float32(w.info()["deq_scale"]) == GOLD[key][1]
        got = H.run_matmul(w, inp["A"], OUT[case["out"]], steps=case["steps"])
    else:
        w = H.pack(np.ascontiguousarray(inp["B"].T) if tr else inp["B"], tr)
        if case.get("raw"):
            got = H.run_matmul(w, inp["A"], capi.S32 if case["kind"] == "s8" else capi.F32)
        else:
            got = H.run_matmul(w, inp["A"], OUT[case["out"]], steps=case["steps"], bias=inp.get("bias"),
                               deq_scale=case.get("deq", 1.0), q_scale=case.get("q", 1.0),
                               q_scale_per_oc=inp.get("q_oc"))
    if case["data"] == "two" or (case["kind"] == "s8" and case.get("raw")):
        assert np.array_equal(got, ref)                       # exact arithmetic: bit-exact
    elif got.dtype == np.int8:
        d = np.abs(got.astype(np.int32) - ref.astype(np.int32))
        assert d.max() <= 1 and (d != 0).mean() < 2e-3         # RNE ties on a last-bit fp32 difference
    elif got.dtype == np.uint16:
        assert H.rel_to_max(bf16_to_f32(got), bf16_to_f32(ref)) < 1e-2
    else:
        assert H.rel_to_max(got, ref) < 1e-5


@pytest.mark.parametrize("name", sorted(gc.matvec_cases()))
def test_matvec_matches_reference(name):
    case = gc.matvec_cases()[name]
    inp = gc.matvec_inputs(case)
    A, b = inp["A"], inp["b"]
    dt = capi.BF16 if case["kind"] == "bf16" else capi.S8
    dA, db = H.Dev(A), H.Dev(b)
    dc = H.Dev(shape=(case["M"],), dtype=np.float32 if dt == capi.BF16 else np.int32)
    capi.matvec(dA.ptr, dt, case["M"], case["K"], A.strides[0], db.ptr, dc.ptr)
    assert np.array_equal(dc.numpy(), GOLD[name])


@pytest.mark.parametrize("name", sorted(gc.mlp_cases()))
def test_mlp_matches_reference(name):
    case = gc.mlp_cases()[name]
    inp = gc.mlp_inputs(case)
    M, K, N = case["M"], case["K"], case["N"]
    mlp = capi.Mlp(inp["gate"].ctypes.data, inp["up"].ctypes.data, inp["down"].ctypes.data, K, N)
    out = np.zeros((M, K), np.uint16)
    mlp.run_host(inp["x"].ctypes.data, inp["x"].strides[0], M, out.ctypes.data, out.strides[0])
    act = np.empty((M, N), np.uint16)
    capi.memcpy(act.ctypes.data, mlp.act_ptr(), act.nbytes)
    assert H.rel_to_max(bf16_to_f32(act), bf16_to_f32(GOLD[name + "/act"])) < 1e-2
    assert H.rel_to_max(bf16_to_f32(out), bf16_to_f32(GOLD[name])) < 1e-2
