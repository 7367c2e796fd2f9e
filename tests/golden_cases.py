"""Seeded case list shared by tests/golden/make_golden.py (which records the reference's outputs) and the tests
(which regenerate the same inputs and compare).  Inputs never enter the fixture file, only outputs do."""
import zlib

import numpy as np

from oracle._common import bf16_bits

DEQUANT, BIAS, GELU, QUANT = 1, 2, 4, 8
F32, BF16, S8 = 0, 1, 2


def _seed(name):
    return zlib.crc32(name.encode())


def fc_cases():
    c = {}
    # tail shapes of the reference's accuracy run, two-valued inputs (exact sums)
    for (M, K, N) in [(16, 65, 32), (16, 69, 32), (32, 64, 5), (128, 96, 16), (2, 337, 271), (22, 320, 256),
                      (705, 320, 257), (735, 337, 271)]:
        for tr in (False, True):
            t = "T" if tr else "N"
            c["fc/bf16/two/%dx%dx%d/%s" % (M, K, N, t)] = dict(kind="bf16", M=M, K=K, N=N, transposeB=tr, data="two",
                                                               raw=True)
            if K >= 64:
                data = "two" if M == 705 else "full"   # int32 noise does not compress: one large full-range case
                c["fc/s8/%s/%dx%dx%d/%s" % (data, M, K, N, t)] = dict(kind="s8", M=M, K=K, N=N, transposeB=tr,
                                                                      data=data, raw=True, nthr=2)
            c["fc/w8/two/%dx%dx%d/%s" % (M, K, N, t)] = dict(kind="w8", M=M, K=K, N=N, transposeB=tr, data="two",
                                                             steps=DEQUANT, out=F32)
    # random data through the post-op combinations
    for (M, K, N) in [(4, 512, 384), (100, 512, 384)]:
        c["fc/bf16/uniform/bias/%d" % M] = dict(kind="bf16", M=M, K=K, N=N, transposeB=False, data="uniform",
                                                steps=BIAS, out=F32, nthr=3)
        c["fc/bf16/uniform/bias_gelu_bf16/%d" % M] = dict(kind="bf16", M=M, K=K, N=N, transposeB=True, data="uniform",
                                                          steps=BIAS | GELU, out=BF16)
        c["fc/s8/full/deq_bias_gelu_quant/%d" % M] = dict(kind="s8", M=M, K=K, N=N, transposeB=False, data="full",
                                                          steps=DEQUANT | BIAS | GELU | QUANT, out=S8, deq=0.0008,
                                                          q=25.0)
        c["fc/s8/full/deq_bias_quant_oc/%d" % M] = dict(kind="s8", M=M, K=K, N=N, transposeB=False, data="full",
                                                        steps=DEQUANT | BIAS | QUANT, out=S8, deq=0.0008, q_oc=True)
        c["fc/s8/full/deq_bias_f32/%d" % M] = dict(kind="s8", M=M, K=K, N=N, transposeB=True, data="full",
                                                   steps=DEQUANT | BIAS, out=F32, deq=0.0008)
        c["fc/w8/normal/deq_bf16/%d" % M] = dict(kind="w8", M=M, K=K, N=N, transposeB=False, data="normal",
                                                 steps=DEQUANT, out=BF16)
        c["fc/w8/int/per_channel/%d" % M] = dict(kind="w8", M=M, K=K, N=N, transposeB=False, data="int127",
                                                 per_channel=True)
    return c


def fc_inputs(case):
    rng = np.random.default_rng(_seed("%(kind)s %(M)d %(K)d %(N)d %(data)s" % case))
    M, K, N = case["M"], case["K"], case["N"]
    d = {}
    if case["kind"] == "s8":
        if case["data"] == "two":
            d["A"] = rng.choice(np.array([-1, 1], np.int8), (M, K)); d["B"] = rng.choice(np.array([-1, 1], np.int8), (K, N))
        else:
            d["A"] = rng.integers(-128, 128, (M, K), dtype=np.int8); d["B"] = rng.integers(-128, 128, (K, N), dtype=np.int8)
    else:
        if case["data"] == "two":
            d["A"] = bf16_bits(rng.choice(np.array([-0.5, 0.5], np.float32), (M, K)))
            d["B"] = bf16_bits(rng.choice(np.array([-0.5, 0.5], np.float32), (K, N)))
        elif case["data"] == "uniform":
            d["A"] = bf16_bits(rng.uniform(-1, 1, (M, K)).astype(np.float32))
            d["B"] = bf16_bits(rng.uniform(-1, 1, (K, N)).astype(np.float32))
        elif case["data"] == "normal":
            d["A"] = bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
            d["B"] = bf16_bits((rng.standard_normal((K, N)) * 0.02).astype(np.float32))
        elif case["data"] == "int127":
            d["A"] = bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
            Wq = rng.integers(-127, 128, (K, N)).astype(np.int8)
            Wq[0, 0] = 127  # absmax 127 -> the reference's quantiser reproduces the integers exactly
            d["Wq"] = Wq
            d["B"] = bf16_bits(Wq.astype(np.float32))
            d["scale"] = rng.uniform(0.001, 0.02, N).astype(np.float32)
    d["bias"] = rng.standard_normal(N).astype(np.float32)
    if case.get("q_oc"):
        d["q_oc"] = rng.uniform(10.0, 40.0, N).astype(np.float32)
    if not (case.get("steps", 0) & BIAS):
        d.pop("bias")
    return d


def matvec_cases():
    c = {}
    for (M, K) in [(901, 80), (901, 96), (256, 128), (64, 32), (64, 100)]:
        c["matvec/bf16/%dx%d" % (M, K)] = dict(kind="bf16", M=M, K=K)
    for (M, K) in [(901, 96), (256, 128), (64, 64), (70, 200)]:
        c["matvec/s8/%dx%d" % (M, K)] = dict(kind="s8", M=M, K=K)
    return c


def matvec_inputs(case):
    rng = np.random.default_rng(_seed("mv %(kind)s %(M)d %(K)d" % case))
    M, K = case["M"], case["K"]
    if case["kind"] == "bf16":
        return dict(A=bf16_bits(rng.choice(np.array([-0.5, 0.5], np.float32), (M, K))),
                    b=bf16_bits(rng.choice(np.array([-0.5, 0.5], np.float32), (K,))))
    return dict(A=rng.integers(-128, 128, (M, K), dtype=np.int8), b=rng.integers(-128, 128, (K,), dtype=np.int8))


def mlp_cases():
    return {
        "mlp/normal/M3": dict(M=3, K=512, N=1024, data="normal"),
        "mlp/normal/M40": dict(M=40, K=512, N=1024, data="normal"),
        "mlp/two/M32": dict(M=32, K=256, N=512, data="two"),
    }


def mlp_inputs(case):
    rng = np.random.default_rng(_seed("mlp %(M)d %(K)d %(N)d %(data)s" % case))
    M, K, N = case["M"], case["K"], case["N"]
    if case["data"] == "two":
        f = lambda s: bf16_bits(rng.choice(np.array([-0.5, 0.5], np.float32), s))
        return dict(x=f((M, K)), gate=f((N, K)), up=f((N, K)), down=f((K, N)))
    return dict(x=bf16_bits(rng.standard_normal((M, K)).astype(np.float32)),
                gate=bf16_bits((rng.standard_normal((N, K)) * 0.02).astype(np.float32)),
                up=bf16_bits((rng.standard_normal((N, K)) * 0.02).astype(np.float32)),
                down=bf16_bits((rng.standard_normal((K, N)) * 0.02).astype(np.float32)))


def activation_points():
    """fixed grid for the GeLU polynomial / SiLU checks, all zones of the reference's GeLU included"""
    x = np.concatenate([np.linspace(-12, 12, 2001), np.array([0.0, 1e-9, -1e-9, 5.0, -5.0, 5.0001, -5.0001, 30.0,
                                                                -30.0, 88.0, -88.0, 100.0, -100.0, 1e-3, -1e-3])])
    x = x.astype(np.float32)
    pad = (-x.size) % 16
    return np.concatenate([x, np.zeros(pad, np.float32)])


def mha_cases():
    """one-token attention of the reference (MHA2Kernels, include/kernels_mha.hpp:89-318): B sequences, H heads (the
    reference has no grouped heads), N cached tokens, head size K, sub-states of bn tokens.  N is a multiple of 8 in
    every case: for other N the reference's own AVX2 kernels leave the textbook result (checked at N = 17, 255, 300,
    700: up to a quarter of max |result|), so those lengths are covered against the float64 restatement only."""
    shapes = [(1, 2, 16, 64, 256), (2, 4, 304, 128, 256), (1, 3, 1000, 128, 256), (2, 2, 704, 64, 128),
              (1, 1, 248, 128, 256), (3, 5, 2048, 128, 256), (1, 2, 520, 32, 64), (2, 8, 8, 128, 256),
              (1, 4, 4096, 64, 512)]
    return {"mha/B%d_H%d_N%d_K%d_bn%d" % s: dict(B=s[0], H=s[1], N=s[2], K=s[3], bn=s[4]) for s in shapes}


def mha_inputs(case):
    """bf16 bit patterns: q [B, H, K], k and v [B, H, N, K] (the reference computes in fp32 on the widened values)"""
    rng = np.random.default_rng(_seed("mha %(B)d %(H)d %(N)d %(K)d" % case))
    B, H, N, K = case["B"], case["H"], case["N"], case["K"]
    return dict(q=bf16_bits((rng.standard_normal((B, H, K)) * 0.5).astype(np.float32)),
                k=bf16_bits((rng.standard_normal((B, H, N, K)) * 0.5).astype(np.float32)),
                v=bf16_bits(rng.standard_normal((B, H, N, K)).astype(np.float32)))
