"""GPU: the benchmark configurations at their FULL sizes, where the CPU oracle would take minutes.

The small-shape tests pin the kernels against the oracle bit for bit; here the same entry points run the shapes the
benchmark is quoted on and are checked against an independent full-size computation on the same GPU (torch fp32 /
fp64 matmuls, not this library) and through properties that do not depend on the size:
  * int8 x int8 accumulators equal the fp64 product exactly (|acc| < 2^53);
  * bf16 paths stay within max|err| <= 1e-2 * max|ref|, the bar of the bf16 paths;
  * the decode kernels (M <= 16) and the GEMM (M > 16) agree on the rows they share;
  * the MLP is positively homogeneous in the down projection: scaling `down` by 2 (exact in bf16) doubles the output
    bit for bit.
The reference builders are plain functions of torch tensors so that a CPU test can run them on tiny shapes.
"""
import numpy as np
import pytest
import torch

from mm_amx_b200 import capi

BAR = 1e-2   # max|err| / max|ref| for bf16 paths


def rel_to_max(got, ref):
    return float((got.float() - ref.float()).abs().max() / ref.float().abs().max())


def mlp_reference(x, gate, up, down):
    """fp32 products, bf16 rounding of the activation and of the output, like the reference's mlp_ref
    (tests/amx-mlp.cpp:811-819)."""
    act = (torch.nn.functional.silu(x.float() @ gate.float().T) * (x.float() @ up.float().T)).to(torch.bfloat16)
    return (act.float() @ down.float().T).to(torch.bfloat16)


def int8_weight_reference(x, wq, scale):
    """bf16 activations x int8 weights, per-output-channel fp32 scale, bf16 output (the fc16m-style decode configuration of the benchmark list)."""
    return ((x.float() @ wq.float().T) * scale[None, :]).to(torch.bfloat16)


def randn_bf16(shape, std, gen, device):
    return (torch.randn(shape, generator=gen, device=device) * std).to(torch.bfloat16)


def run_mlp(x, gate, up, down):
    M, K = x.shape
    mlp = capi.Mlp(gate.data_ptr(), up.data_ptr(), down.data_ptr(), K, gate.shape[0])
    out = torch.empty((M, K), dtype=torch.bfloat16, device=x.device)
    mlp.run(x.data_ptr(), K * 2, M, out.data_ptr(), K * 2)
    capi.sync_check()
    return out, mlp


@pytest.mark.gpu
def test_config1_bf16_linear_256x4096x4096_bias():
    dev = torch.device("cuda")
    g = torch.Generator(device=dev); g.manual_seed(1001)
    M, K, N = 256, 4096, 4096
    A = (torch.rand((M, K), generator=g, device=dev) * 2 - 1).to(torch.bfloat16)
    B = (torch.rand((N, K), generator=g, device=dev) * 2 - 1).to(torch.bfloat16)      # [N, K]: transposeB
    bias = torch.randn(N, generator=g, device=dev)
    w = capi.Weight(B.data_ptr(), capi.BF16, K, N, K * 2, True)
    C = torch.empty((M, N), dtype=torch.float32, device=dev)
    ep = capi.make_epilogue(C.data_ptr(), N * 4, capi.F32, capi.STEP_BIAS, bias.data_ptr())
    w.matmul(A.data_ptr(), capi.BF16, M, K, K * 2, ep)
    capi.sync_check()
    ref = A.float() @ B.float().T + bias[None, :]
    assert rel_to_max(C, ref) < 1e-4          # fp32 output: far inside the bf16 bar


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N", [(2048, 4096, 22016), (2048, 11008, 4096), (4096, 8192, 7168), (4096, 8192, 14336),
                                   (3300, 8192, 5888)])
def test_llama_shaped_gemms_against_fp32(M, K, N):
    """the last three are taken in panels of 8 row tiles (x over 48 MB) and leave a ragged last round that a K-split
    launch takes over: the bottom four tiles of the last column block, the last column block of the last panel, and a
    short last panel (13 row tiles: 8 + 5)"""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev); g.manual_seed(M + N)
    A = randn_bf16((M, K), 1.0, g, dev)
    B = randn_bf16((N, K), 0.02, g, dev)
    w = capi.Weight(B.data_ptr(), capi.BF16, K, N, K * 2, True)
    C = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    ep = capi.make_epilogue(C.data_ptr(), N * 2, capi.BF16)
    w.matmul(A.data_ptr(), capi.BF16, M, K, K * 2, ep)
    capi.sync_check()
    ref = A.float() @ B.float().T
    assert rel_to_max(C, ref) < BAR
    # decode kernel and GEMM agree on shared rows (both round the same fp32 sums to bf16, up to summation order)
    C4 = torch.empty((4, N), dtype=torch.bfloat16, device=dev)
    ep4 = capi.make_epilogue(C4.data_ptr(), N * 2, capi.BF16)
    w.matmul(A.data_ptr(), capi.BF16, 4, K, K * 2, ep4)
    capi.sync_check()
    assert rel_to_max(C4, ref[:4]) < BAR
    assert rel_to_max(C4, C[:4]) < BAR


@pytest.mark.gpu
def test_config4_int8_2048x4096x4096_exact():
    dev = torch.device("cuda")
    g = torch.Generator(device=dev); g.manual_seed(1004)
    M, K, N = 2048, 4096, 4096
    A = torch.randint(-128, 128, (M, K), generator=g, device=dev, dtype=torch.int8)
    B = torch.randint(-128, 128, (N, K), generator=g, device=dev, dtype=torch.int8)
    w = capi.Weight(B.data_ptr(), capi.S8, K, N, K, True)
    C = torch.empty((M, N), dtype=torch.int32, device=dev)
    ep = capi.make_epilogue(C.data_ptr(), N * 4, capi.S32)
    w.matmul(A.data_ptr(), capi.S8, M, K, K, ep)
    capi.sync_check()
    ref = (A.double() @ B.double().T).to(torch.int64)      # exact: |acc| <= 2^26
    assert torch.equal(C.to(torch.int64), ref)


@pytest.mark.gpu
def test_config4_int8_2048x4096x4096_quantised_postops():
    """dequantise by sA * sB[n], add bias -> fp32; then requantise to int8 with a q_scale that saturates about 1 % of the
    outputs (round to nearest even + saturation, kernels_amx.hpp:631-664).  Reference: the exact int32 accumulators (fp64
    product) pushed through the same fp32 steps in torch."""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev); g.manual_seed(2004)
    M, K, N = 2048, 4096, 4096
    A = torch.randint(-128, 128, (M, K), generator=g, device=dev, dtype=torch.int8)
    B = torch.randint(-128, 128, (N, K), generator=g, device=dev, dtype=torch.int8)
    sA = 0.013
    sB = torch.rand(N, generator=g, device=dev) * 0.049 + 0.001
    bias = torch.randn(N, generator=g, device=dev)
    w = capi.Weight(B.data_ptr(), capi.S8, K, N, K, True)
    acc = (A.double() @ B.double().T).to(torch.int32)
    ref_f = (acc.float() * (np.float32(sA) * sB)[None, :]) + bias[None, :]
    Cf = torch.empty((M, N), dtype=torch.float32, device=dev)
    ep = capi.make_epilogue(Cf.data_ptr(), N * 4, capi.F32, capi.STEP_DEQUANT | capi.STEP_BIAS, bias.data_ptr(), sA,
                            sB.data_ptr())
    w.matmul(A.data_ptr(), capi.S8, M, K, K, ep)
    capi.sync_check()
    # same fp32 operations in the same order; only the fused multiply-add contraction of `* scale + bias` may differ
    assert rel_to_max(Cf, ref_f) < 1e-6
    q = float(127.0 / (2.576 * ref_f.std().item()))          # |z| > 2.576 sigma: about 1 % of a normal distribution
    C8 = torch.empty((M, N), dtype=torch.int8, device=dev)
    ep8 = capi.make_epilogue(C8.data_ptr(), N, capi.S8, capi.STEP_DEQUANT | capi.STEP_BIAS | capi.STEP_QUANT,
                             bias.data_ptr(), sA, sB.data_ptr(), q)
    w.matmul(A.data_ptr(), capi.S8, M, K, K, ep8)
    capi.sync_check()
    ref8 = torch.clamp(torch.round(Cf * np.float32(q)), -128, 127).to(torch.int8)     # torch.round: half to even
    sat = float(((ref8 == 127) | (ref8 == -128)).float().mean().item())
    assert 0.002 < sat < 0.05, sat
    assert torch.equal(C8, ref8)


@pytest.mark.gpu
def test_config5_llama70b_mlp_whole_on_one_gpu():
    """tensor-parallel size 1, M = 4096: the shape the scaling run starts from.  Rows 0..63 against torch fp32 on the
    GPU; the decode kernel (M = 1, 16) and the GEMM path must agree on the rows they share."""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev); g.manual_seed(3005)
    H, I, M = 8192, 28672, 4096
    gate, up, down = randn_bf16((I, H), 0.02, g, dev), randn_bf16((I, H), 0.02, g, dev), randn_bf16((H, I), 0.02, g, dev)
    x = randn_bf16((M, H), 1.0, g, dev)
    mlp = capi.Mlp(gate.data_ptr(), up.data_ptr(), down.data_ptr(), H, I)
    out = torch.empty((M, H), dtype=torch.bfloat16, device=dev)
    mlp.run(x.data_ptr(), H * 2, M, out.data_ptr(), H * 2)
    capi.sync_check()
    for r0 in (0, M - 64):
        assert rel_to_max(out[r0:r0 + 64], mlp_reference(x[r0:r0 + 64], gate, up, down)) < BAR
    for Md in (1, 16, 128):
        o = torch.empty((Md, H), dtype=torch.bfloat16, device=dev)
        mlp.run(x.data_ptr(), H * 2, Md, o.data_ptr(), H * 2)
        capi.sync_check()
        assert rel_to_max(o, out[:Md]) < BAR


@pytest.mark.gpu
@pytest.mark.parametrize("N", [4096, 11008])
@pytest.mark.parametrize("M", [1, 4, 16])
def test_config3_int8_weight_gemv(M, N):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev); g.manual_seed(1003 + M + N)
    K = 4096
    x = randn_bf16((M, K), 1.0, g, dev)
    wq = torch.randint(-127, 128, (N, K), generator=g, device=dev, dtype=torch.int8)
    scale = torch.rand(N, generator=g, device=dev) * 0.019 + 0.001
    w = capi.Weight(wq.data_ptr(), capi.S8, K, N, K, True, capi.PACK_INT8_CHANNEL, scale.data_ptr())
    C = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    ep = capi.make_epilogue(C.data_ptr(), N * 2, capi.BF16, capi.STEP_DEQUANT)
    w.matmul(x.data_ptr(), capi.BF16, M, K, K * 2, ep)
    capi.sync_check()
    assert rel_to_max(C, int8_weight_reference(x, wq, scale)) < BAR


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 16, 256, 2048])
def test_config2_llama7b_mlp(M):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev); g.manual_seed(1002)
    H, I = 4096, 11008
    gate, up, down = randn_bf16((I, H), 0.02, g, dev), randn_bf16((I, H), 0.02, g, dev), randn_bf16((H, I), 0.02, g, dev)
    x = randn_bf16((M, H), 1.0, g, dev)
    out, _ = run_mlp(x, gate, up, down)
    assert rel_to_max(out, mlp_reference(x, gate, up, down)) < BAR
    # scaling the down projection by 2 is exact in bf16 and in every fp32 sum: the output doubles bit for bit
    out2, _ = run_mlp(x, gate, up, (down.float() * 2).to(torch.bfloat16))
    assert torch.equal(out2.float(), out.float() * 2)


@pytest.mark.gpu
@pytest.mark.parametrize("M", [16, 1024])
def test_config5_llama70b_mlp_shard_of_8(M):
    """one rank's share at tensor-parallel size 8 (rows of gate/up and columns of down), fp32 contribution"""
    dev = torch.device("cuda")
    g = torch.Generator(device=dev); g.manual_seed(1005)
    H, Is = 8192, 28672 // 8
    gate, up, down = randn_bf16((Is, H), 0.02, g, dev), randn_bf16((Is, H), 0.02, g, dev), randn_bf16((H, Is), 0.02, g, dev)
    x = randn_bf16((M, H), 1.0, g, dev)
    mlp = capi.Mlp(gate.data_ptr(), up.data_ptr(), down.data_ptr(), H, Is)
    part = torch.empty((M, H), dtype=torch.float32, device=dev)
    mlp.run_partial(x.data_ptr(), H * 2, M, part.data_ptr(), capi.F32, H * 4)
    capi.sync_check()
    act = (torch.nn.functional.silu(x.float() @ gate.float().T) * (x.float() @ up.float().T)).to(torch.bfloat16)
    ref = act.float() @ down.float().T
    assert rel_to_max(part, ref) < BAR


def test_reference_builders_on_cpu():
    """the reference functions above, on tiny CPU tensors (no GPU, no library call): shapes, dtypes, homogeneity"""
    g = torch.Generator(); g.manual_seed(0)
    x = randn_bf16((3, 64), 1.0, g, "cpu")
    gate, up, down = randn_bf16((96, 64), 0.1, g, "cpu"), randn_bf16((96, 64), 0.1, g, "cpu"), randn_bf16((64, 96), 0.1, g, "cpu")
    ref = mlp_reference(x, gate, up, down)
    assert ref.shape == (3, 64) and ref.dtype == torch.bfloat16
    ref2 = mlp_reference(x, gate, up, (down.float() * 2).to(torch.bfloat16))
    assert torch.equal(ref2.float(), ref.float() * 2)
    wq = torch.randint(-127, 128, (32, 64), generator=g, dtype=torch.int8)
    scale = torch.rand(32, generator=g) * 0.019 + 0.001
    r = int8_weight_reference(x, wq, scale)
    assert r.shape == (3, 32) and r.dtype == torch.bfloat16
    assert rel_to_max(r, r) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["int8", "int4"])
def test_quantised_decode_large_matrix_is_deterministic_and_right(mode):
    """8192 x 28672 with quantised weights at M = 16: every CTA walks several activation chunks (pre-converted images
    copied asynchronously into alternating buffers) and most row blocks are summed across CTAs through the scratch.
    Twenty launches must give identical bits (a race in the ring or in the chunk buffers shows as a flicker), and rows
    checked against a float64 product of the dequantised weights."""
    import torch
    torch.manual_seed(5)
    M, K, N = 16, 8192, 28672
    x = torch.randn((M, K), device="cuda").to(torch.bfloat16)
    if mode == "int8":
        Wq = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda")
        sc = torch.rand(N, device="cuda") * 0.019 + 0.001
        w = capi.Weight(Wq.data_ptr(), capi.S8, K, N, K, True, capi.PACK_INT8_CHANNEL, sc.data_ptr())
        deq_rows = lambda rows: Wq[rows].double() * sc[rows].double()[:, None]
    else:
        W = (torch.randn((N, K), device="cuda") * 0.02).to(torch.bfloat16)
        w = capi.Weight(W.data_ptr(), capi.BF16, K, N, K * 2, True, capi.PACK_INT4_GROUP)
        q = torch.empty((N, K), dtype=torch.int8, device="cuda")
        w.unpack(q.data_ptr(), K)
        gs = np.zeros((N, K // 128), np.float32)
        w.group_scales(gs.ctypes.data, gs.strides[0])
        gs_t = torch.from_numpy(gs).cuda()
        deq_rows = lambda rows: q[rows].double() * gs_t[rows].double().repeat_interleave(128, dim=1)
    out = torch.empty((M, N), dtype=torch.float32, device="cuda")
    ep = capi.make_epilogue(out.data_ptr(), N * 4, capi.F32, capi.STEP_DEQUANT)
    first = None
    for it in range(20):
        out.fill_(float("nan"))
        w.matmul(x.data_ptr(), capi.BF16, M, K, K * 2, ep)
        capi.sync_check()
        cur = out.clone()
        if first is None:
            first = cur
        else:
            assert torch.equal(first.view(torch.int32), cur.view(torch.int32)), "launch %d differs from the first" % it
    rows = torch.arange(0, N, 97, device="cuda")
    ref = x.double() @ deq_rows(rows).T
    err = (first[:, rows].double() - ref).abs().max() / ref.abs().max()
    assert err.item() < 1e-5
