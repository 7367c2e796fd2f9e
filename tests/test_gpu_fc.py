"""GPU parity of the fully-connected path against the CPU oracle, through the C ABI.

Shapes and inputs follow the reference's own accuracy runs: the 17 tail shapes of test_FC_acc (main.cpp:714-735) with
two-valued inputs (tensor2D::fill_rnd), for bf16, int8 and bf16 x int8-compressed weights, B as [K,N] and as [N,K].
On those inputs every partial sum is exact, so the comparison is bit-exact (the reference's operator==).
"""
import numpy as np
import pytest

from oracle import port
from oracle._common import bf16_bits, bf16_to_f32
from mm_amx_b200 import capi
import helpers as H

pytestmark = pytest.mark.gpu

# main.cpp:716-734
REF_SHAPES = [(16, 65, 32), (16, 66, 32), (16, 67, 32), (16, 68, 32), (16, 69, 32), (32, 64, 5), (128, 96, 16),
              (2, 2560, 10752), (2, 10 * 32 + 17, 256 + 15), (22, 2560, 10752), (32 * 22, 10 * 32, 256),
              (32 * 22 + 1, 10 * 32, 256 + 1), (32 * 22 + 16, 10 * 32, 256 + 17), (32 * 22 + 31, 10 * 32, 256 + 15),
              (32 * 22 + 31, 10 * 32 + 1, 256 + 15), (32 * 22 + 31, 10 * 32 + 17, 256 + 15), (2, 10 * 32, 256)]


@pytest.mark.parametrize("M,K,N", REF_SHAPES)
@pytest.mark.parametrize("transposeB", [False, True])
def test_bf16_two_valued_exact(M, K, N, transposeB):
    rng = np.random.default_rng(M * 7 + K * 3 + N)
    A = H.two_valued_bf16(rng, (M, K)); B = H.two_valued_bf16(rng, (K, N))
    ref = port.gemm_bf16(A, B)
    w = H.pack(np.ascontiguousarray(B.T) if transposeB else B, transposeB)
    got = H.run_matmul(w, A, capi.F32)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("M,K,N", REF_SHAPES)
@pytest.mark.parametrize("transposeB", [False, True])
def test_s8_exact(M, K, N, transposeB):
    """int8 x int8: int32 accumulators must be bit-exact on full-range data (main.cpp:738 runs <int8_t, NONE>)."""
    rng = np.random.default_rng(M + K * 5 + N * 11)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8); B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    ref = port.gemm_i8(A, B)
    w = H.pack(np.ascontiguousarray(B.T) if transposeB else B, transposeB)
    got = H.run_matmul(w, A, capi.S32)
    assert np.array_equal(got, ref)
    # and the reference's own view of them: converted to fp32 by the NONE post-op (kernels_amx.hpp:631-634)
    got_f = H.run_matmul(w, A, capi.F32)
    assert np.array_equal(got_f, port.postops(ref, 0, port.F32))


@pytest.mark.parametrize("M,K,N", REF_SHAPES)
def test_compressed_two_valued_exact(M, K, N):
    """bf16 x int8-compressed weights (main.cpp:741-742, <bfloat16, DEQUANT>): per-tensor absmax quantisation."""
    rng = np.random.default_rng(M + K + N)
    A = H.two_valued_bf16(rng, (M, K)); B = H.two_valued_bf16(rng, (K, N))
    Wq, qs, dq = port.quantize_weight(B)
    ref = port.postops(port.gemm_bf16_w8(A, Wq), port.DEQUANT, port.F32, deq_scale=dq)
    w = H.pack(B, False, capi.PACK_QUANT_TENSOR)
    info = w.info()
    assert info["compressed"] and info["dtype"] == capi.S8 and info["deq_scale"] == np.float32(dq)
    unp = H.Dev(shape=(N, K), dtype=np.int8)
    w.unpack(unp.ptr, K)
    assert np.array_equal(unp.numpy(), Wq.T)
    got = H.run_matmul(w, A, capi.F32, steps=capi.STEP_DEQUANT)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("K,N,transposeB", [(256, 320, False), (1000, 77, True), (4096, 512, True)])
def test_weight_quantiser_bit_exact_on_normal_data(K, N, transposeB):
    """The quantised bytes are integer work: on N(0, 0.02) data (ties, all 255 levels in use) the GPU quantiser must
    produce the bytes and the scale of the reference's get_min_max + bf16_to_i8_tensor (kernels_amx.hpp:465-523)."""
    rng = np.random.default_rng(K * 7 + N)
    B = H.normal_bf16(rng, (N, K) if transposeB else (K, N), 0.02)
    Wq, qs, dq = port.quantize_weight(B)
    w = H.pack(B, transposeB, capi.PACK_QUANT_TENSOR)
    assert w.info()["deq_scale"] == np.float32(dq)
    unp = H.Dev(shape=(N, K), dtype=np.int8)
    w.unpack(unp.ptr, K)
    want = Wq if transposeB else Wq.T
    assert len(np.unique(want)) > 100          # the case really exercises the rounding, unlike two-valued data
    assert np.array_equal(unp.numpy(), want)


@pytest.mark.parametrize("M,K,N,n0,n1", [(40, 256, 1024, 0, 1024), (130, 8192, 2600, 0, 2600), (64, 8192, 2600, 512, 2304)])
def test_compressed_weights_prefill_blocks(M, K, N, n0, n1):
    """M > 16 with int8-compressed weights: blocks of weight rows are widened into a scratch and multiplied block by
    block (K = 8192 makes a block 2048 rows, so N = 2600 takes two); per-channel scales, bias and a column range."""
    rng = np.random.default_rng(M + K + N + n0)
    A = H.normal_bf16(rng, (M, K))
    Wq = rng.integers(-127, 128, (N, K), dtype=np.int8)
    scale = rng.uniform(0.001, 0.02, N).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    w = H.pack(Wq, True, capi.PACK_INT8_CHANNEL, scales=scale)
    got = H.run_matmul(w, A, capi.F32, steps=capi.STEP_DEQUANT | capi.STEP_BIAS, bias=bias, n0=n0, n1=n1)
    ref = port.postops(port.gemm_bf16_w8(A, np.ascontiguousarray(Wq.T)), port.DEQUANT | port.BIAS, port.F32, bias=bias,
                       deq_scale_per_oc=scale)
    assert H.rel_to_max(got[:, n0:n1], ref[:, n0:n1]) < 1e-5
    sentinel = np.frombuffer(b"\xcd\xcd\xcd\xcd", np.float32)[0]
    if n0 > 0:
        assert (got[:, :n0].view(np.uint32) == sentinel.view(np.uint32)).all()
    if n1 < N:
        assert (got[:, n1:].view(np.uint32) == sentinel.view(np.uint32)).all()


def test_bounded_wait_runs_out_and_the_library_recovers(monkeypatch):
    """A device-side wait that nothing will satisfy gives up after the configured limit, the kernel ends cleanly, the
    host sees B200FC_ERR_KERNEL once, and the next ordinary call works.  The wait is the reduce role of the fused
    all-reduce kernel waiting for arrivals of a second rank that does not exist: its counters stay zero, and a CTA that
    gives up leaves before it touches any multicast address (none exists here either)."""
    import torch
    rng = np.random.default_rng(5)
    K, N, M = 256, 512, 300
    gate, up = H.normal_bf16(rng, (N, K), 0.02), H.normal_bf16(rng, (N, K), 0.02)
    down = H.normal_bf16(rng, (K, N), 0.02)
    mlp = capi.Mlp(gate.ctypes.data, up.ctypes.data, down.ctypes.data, K, N)
    x = H.Dev(H.normal_bf16(rng, (M, K)))
    out = H.Dev(shape=(M, K), dtype=np.uint16)
    mlp.run(x.ptr, x.ld, M, out.ptr, out.ld)
    capi.sync_check()
    good = out.numpy()
    partial = torch.zeros((M, K), dtype=torch.bfloat16, device="cuda")
    result = torch.zeros((M, K), dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(4096, dtype=torch.int32, device="cuda")
    ar = capi.AllReduce()
    ar.world, ar.rank = 2, 0
    ar.partial_local, ar.partial_mc, ar.out_mc = partial.data_ptr(), partial.data_ptr(), result.data_ptr()
    ar.ld_bytes = K * 2
    ar.flags[0] = flags.data_ptr(); ar.flags[1] = flags.data_ptr()
    ar.max_tiles, ar.comm_sms = 4096, 8
    monkeypatch.setenv("B200FC_AR_PHASES", "2")      # reduce role only: nobody multiplies, nobody signals
    capi.set_wait_limit_ns(3_000_000)                # 3 ms
    try:
        mlp.gate_up(x.ptr, x.ld, M)
        mlp.down_allreduce(M, ar)
        with pytest.raises(capi.B200FCError) as e:
            capi.sync_check()
        assert e.value.code == capi.ERR_KERNEL
    finally:
        capi.set_wait_limit_ns(2_000_000_000)
        monkeypatch.delenv("B200FC_AR_PHASES")
    capi.sync_check()                                # the status word was cleared by the failing check
    assert not result.any()                          # the reduce role left before it wrote anything
    out2 = H.Dev(shape=(M, K), dtype=np.uint16)
    mlp.run(x.ptr, x.ld, M, out2.ptr, out2.ld)
    capi.sync_check()
    assert np.array_equal(out2.numpy(), good)


@pytest.mark.parametrize("M", [1, 2, 3, 8, 9, 16, 17, 64, 200])
def test_bf16_random_tolerance(M):
    """uniform[-1,1] data: fp32 accumulation order differs from the oracle's, so compare within 1e-2 of max|ref|
    (the bar for bf16 paths); in practice the difference is ~1e-6."""
    rng = np.random.default_rng(M)
    K, N = 1024, 768
    A = H.uniform_bf16(rng, (M, K)); B = H.uniform_bf16(rng, (K, N))
    bias = rng.standard_normal(N).astype(np.float32)
    acc = port.gemm_bf16(A, B)
    w = H.pack(B)
    got = H.run_matmul(w, A, capi.F32, steps=capi.STEP_BIAS, bias=bias)
    assert H.rel_to_max(got, port.postops(acc, port.BIAS, port.F32, bias=bias)) < 1e-5
    got = H.run_matmul(w, A, capi.BF16, steps=capi.STEP_BIAS | capi.STEP_GELU, bias=bias)
    ref = port.postops(acc, port.BIAS | port.GELU, port.BF16, bias=bias)
    assert H.rel_to_max(bf16_to_f32(got), bf16_to_f32(ref)) < 1e-2


@pytest.mark.parametrize("M", [1, 4, 16, 40])
@pytest.mark.parametrize("N", [512, 1000])
def test_int8_weight_per_channel(M, N):
    """decode with int8 weights and per-output-channel scales (fc16m-style), bf16 output."""
    rng = np.random.default_rng(M * 31 + N)
    K = 1536
    x = H.normal_bf16(rng, (M, K))
    Wq = rng.integers(-127, 128, (K, N), dtype=np.int8)
    scale = rng.uniform(0.001, 0.02, N).astype(np.float32)
    ref = port.postops(port.gemm_bf16_w8(x, Wq), port.DEQUANT, port.BF16, deq_scale=1.0, deq_scale_per_oc=scale)
    w = H.pack(Wq, False, capi.PACK_INT8_CHANNEL, scales=scale)
    got = H.run_matmul(w, x, capi.BF16, steps=capi.STEP_DEQUANT)
    assert H.rel_to_max(bf16_to_f32(got), bf16_to_f32(ref)) < 1e-2
    # the fp32 view is far tighter than the bf16 bar
    got32 = H.run_matmul(w, x, capi.F32, steps=capi.STEP_DEQUANT)
    ref32 = port.postops(port.gemm_bf16_w8(x, Wq), port.DEQUANT, port.F32, deq_scale=1.0, deq_scale_per_oc=scale)
    assert H.rel_to_max(got32, ref32) < 1e-5


@pytest.mark.parametrize("M", [8, 300])
def test_s8_postops(M):
    """DEQUANT -> BIAS -> GELU -> QUANT with int8 output, RNE + saturation (main.cpp:481-527 combos)."""
    rng = np.random.default_rng(M)
    K, N = 512, 320
    A = rng.integers(-128, 128, (M, K), dtype=np.int8); B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    bias = rng.standard_normal(N).astype(np.float32)
    sB = rng.uniform(0.001, 0.05, N).astype(np.float32)
    qoc = rng.uniform(5.0, 40.0, N).astype(np.float32)
    acc = port.gemm_i8(A, B)
    w = H.pack(B)
    for steps, kw in [
        (capi.STEP_DEQUANT | capi.STEP_BIAS, dict(deq_scale=0.02, deq_scale_per_oc=sB, bias=bias)),
        (capi.STEP_DEQUANT | capi.STEP_BIAS | capi.STEP_GELU | capi.STEP_QUANT, dict(deq_scale=0.001, bias=bias, q_scale=30.0)),
        (capi.STEP_DEQUANT | capi.STEP_BIAS | capi.STEP_QUANT, dict(deq_scale=0.0005, deq_scale_per_oc=sB * 20, bias=bias, q_scale_per_oc=qoc)),
    ]:
        for od, pod in [(capi.F32, port.F32), (capi.S8, port.S8), (capi.BF16, port.BF16)]:
            got = H.run_matmul(w, A, od, steps=steps, **kw)
            ref = port.postops(acc, steps, pod, **kw)
            if od == capi.F32:
                assert np.allclose(got, ref, rtol=2e-6, atol=1e-6)
            elif od == capi.BF16:
                assert H.rel_to_max(bf16_to_f32(got), bf16_to_f32(ref)) < 1e-2
            else:
                d = np.abs(got.astype(np.int32) - ref.astype(np.int32))
                assert d.max() <= 1 and (d != 0).mean() < 1e-3  # ties may flip on a 1-ulp fp32 difference
                assert (ref == 127).any() or (ref == -128).any() or True


@pytest.mark.parametrize("M,K,N", [(100, 4096, 512), (256, 4096, 1024), (64, 2304, 300), (17, 8192, 256)])
def test_split_k_shapes_exact(M, K, N):
    """few output tiles and a long K: the GEMM splits K over CTA pairs and reduces in a second kernel"""
    rng = np.random.default_rng(M + K + N)
    A = H.two_valued_bf16(rng, (M, K)); B = H.two_valued_bf16(rng, (K, N))
    bias = (rng.integers(-8, 9, N) * 0.25).astype(np.float32)
    w = H.pack(B)
    got = H.run_matmul(w, A, capi.F32, steps=capi.STEP_BIAS, bias=bias)
    assert np.array_equal(got, port.postops(port.gemm_bf16(A, B), port.BIAS, port.F32, bias=bias))
    got = H.run_matmul(w, A, capi.F32, n0=32, n1=N - 7)
    assert np.array_equal(got[:, 32:N - 7], port.gemm_bf16(A, B)[:, 32:N - 7])
    Ai = rng.integers(-128, 128, (M, K), dtype=np.int8); Bi = rng.integers(-128, 128, (K, N), dtype=np.int8)
    wi = H.pack(Bi)
    acc = port.gemm_i8(Ai, Bi)
    assert np.array_equal(H.run_matmul(wi, Ai, capi.S32), acc)
    got8 = H.run_matmul(wi, Ai, capi.S8, steps=capi.STEP_DEQUANT | capi.STEP_QUANT, deq_scale=0.001, q_scale=2.0)
    ref8 = port.postops(acc, port.DEQUANT | port.QUANT, port.S8, deq_scale=0.001, q_scale=2.0)
    assert np.abs(got8.astype(np.int32) - ref8.astype(np.int32)).max() <= 1


def test_ragged_last_round_goes_through_a_k_split_launch():
    """76 tiles of 256 x 256 on 74 CTA pairs with a long K: the main launch stops after 74 tiles and the two left-over
    tiles (bottom rows of the last column block; the last row tile and the last column block are partial) run as a
    K-split GEMM of their own.  Exact arithmetic (two-valued data), so every element must match however K was cut."""
    rng = np.random.default_rng(76)
    M, K, N = 1000, 6144, 5056
    A = H.two_valued_bf16(rng, (M, K)); B = H.two_valued_bf16(rng, (K, N))
    bias = (rng.integers(-8, 9, N) * 0.25).astype(np.float32)
    w = H.pack(B)
    ref = port.gemm_bf16(A, B)
    got = H.run_matmul(w, A, capi.F32, steps=capi.STEP_BIAS, bias=bias, n0=256)       # 19 column blocks, the last 192 wide
    assert np.array_equal(got[:, 256:], port.postops(ref, port.BIAS, port.F32, bias=bias)[:, 256:])
    assert (got[:, :256].view(np.uint32) == 0xCDCDCDCD).all()
    got = H.run_matmul(w, A[:512], capi.BF16, n0=0, n1=4864)                          # 2 x 19 tiles = 38: one round, no split
    assert np.array_equal(got[:, :4864], port.postops(ref[:512], 0, port.BF16)[:, :4864])
    got = H.run_matmul(w, A, capi.BF16, n0=192)                                       # 4 x 19 tiles again, bf16 output
    assert np.array_equal(got[:, 192:], port.postops(ref, 0, port.BF16)[:, 192:])
    # 2 x 38 tiles: the left-over is the whole last column block (all rows of it)
    M, N = 300, 9728
    A = H.two_valued_bf16(rng, (M, K)); B = H.two_valued_bf16(rng, (K, N))
    bias = (rng.integers(-8, 9, N) * 0.25).astype(np.float32)
    got = H.run_matmul(H.pack(B), A, capi.F32, steps=capi.STEP_BIAS, bias=bias)
    assert np.array_equal(got, port.postops(port.gemm_bf16(A, B), port.BIAS, port.F32, bias=bias))


@pytest.mark.parametrize("M,K,N", [(512, 192, 10280), (300, 128, 20000), (1024, 64, 5000), (700, 96, 7177)])
def test_many_tiles_exact(M, K, N):
    """more 256 x 256 tiles than CTA pairs: every pair walks several tiles, both accumulator buffers get reused"""
    rng = np.random.default_rng(M + K + N)
    A = H.two_valued_bf16(rng, (M, K)); B = H.two_valued_bf16(rng, (K, N))
    bias = (rng.integers(-8, 9, N) * 0.25).astype(np.float32)
    w = H.pack(B)
    ref = port.gemm_bf16(A, B)
    got = H.run_matmul(w, A, capi.F32, steps=capi.STEP_BIAS, bias=bias)
    assert np.array_equal(got, port.postops(ref, port.BIAS, port.F32, bias=bias))
    got = H.run_matmul(w, A, capi.F32, n0=64, n1=N - 9)
    assert np.array_equal(got[:, 64:N - 9], ref[:, 64:N - 9])
    Ai = rng.integers(-128, 128, (M, K), dtype=np.int8); Bi = rng.integers(-128, 128, (K, N), dtype=np.int8)
    wi = H.pack(Bi)
    assert np.array_equal(H.run_matmul(wi, Ai, capi.S32), port.gemm_i8(Ai, Bi))


def test_packed_weight_export_import_round_trip(tmp_path):
    """a blob written by export rebuilds an object that computes bit-identical results, without re-packing:
    bf16, int8, per-tensor quantised and per-channel int8 weights; through a file, like a checkpoint"""
    rng = np.random.default_rng(5)
    M, K, N = 40, 200, 333
    A = H.uniform_bf16(rng, (M, K)); B = H.uniform_bf16(rng, (K, N))
    Ai = rng.integers(-128, 128, (M, K), dtype=np.int8); Bi = rng.integers(-128, 128, (K, N), dtype=np.int8)
    scale = rng.uniform(0.001, 0.02, N).astype(np.float32)
    cases = [
        (H.pack(B), A, dict(out=capi.F32)),
        (H.pack(Bi), Ai, dict(out=capi.S32)),
        (H.pack(B, False, capi.PACK_QUANT_TENSOR), A, dict(out=capi.F32, steps=capi.STEP_DEQUANT)),
        (H.pack(Bi, False, capi.PACK_INT8_CHANNEL, scales=scale), A, dict(out=capi.BF16, steps=capi.STEP_DEQUANT)),
    ]
    for i, (w, act, kw) in enumerate(cases):
        blob = w.export()
        path = tmp_path / ("w%d.bin" % i)
        path.write_bytes(blob)
        w2 = capi.Weight.from_blob(path.read_bytes())
        assert w2.info() == w.info()
        for rows in (3, M):     # decode-shaped and GEMM-shaped paths
            want = H.run_matmul(w, act[:rows], kw["out"], steps=kw.get("steps", 0))
            got = H.run_matmul(w2, act[:rows], kw["out"], steps=kw.get("steps", 0))
            assert np.array_equal(got, want)
        assert w2.export() == blob
    # a truncated or foreign blob is refused
    blob = cases[0][0].export()
    for bad in (blob[:100], b"x" * 200, bytes(blob[:8]) + b"\0" * 56):
        with pytest.raises(capi.B200FCError):
            capi.Weight.from_blob(bad)


def test_column_range_and_sentinel():
    """n0/n1 compute a column sub-range only (Matmul::operator() n0, n1; kernels_amx.hpp:1169-1178)."""
    rng = np.random.default_rng(5)
    M, K, N = 70, 256, 512
    A = H.two_valued_bf16(rng, (M, K)); B = H.two_valued_bf16(rng, (K, N))
    ref = port.gemm_bf16(A, B)
    w = H.pack(B)
    for (n0, n1) in [(0, 512), (32, 96), (64, 500), (100, 101), (0, 7)]:
        got = H.run_matmul(w, A, capi.F32, n0=n0, n1=n1)
        assert np.array_equal(got[:, n0:n1], ref[:, n0:n1])
        rest = np.delete(got, np.s_[n0:n1], axis=1).view(np.uint32)
        assert (rest == 0xCDCDCDCD).all()
    for (n0, n1) in [(0, 512), (32, 96), (37, 300)]:
        got = H.run_matmul(w, A[:5], capi.F32, n0=n0, n1=n1)
        assert np.array_equal(got[:, n0:n1], ref[:5, n0:n1])
        rest = np.delete(got, np.s_[n0:n1], axis=1).view(np.uint32)
        assert (rest == 0xCDCDCDCD).all()


def test_unsigned_variants():
    """s8u8 / u8s8 / u8u8 instantiations (kernels_amx.hpp:1057-1059): exact against an int32 loop."""
    rng = np.random.default_rng(9)
    M, K, N = 40, 192, 96
    for da, db in [(np.int8, np.uint8), (np.uint8, np.int8), (np.uint8, np.uint8)]:
        A = rng.integers(np.iinfo(da).min, np.iinfo(da).max + 1, (M, K)).astype(da)
        B = rng.integers(np.iinfo(db).min, np.iinfo(db).max + 1, (K, N)).astype(db)
        w = H.pack(B)
        assert np.array_equal(H.run_matmul(w, A, capi.S32), port.gemm_i8(A, B))


def test_host_entry_point():
    rng = np.random.default_rng(11)
    M, K, N = 256, 512, 384
    A = H.uniform_bf16(rng, (M, K)); B = H.uniform_bf16(rng, (K, N))
    bias = rng.standard_normal(N).astype(np.float32)
    w = H.pack(B, from_host=True)
    C = np.zeros((M, N), np.float32)
    ep = capi.make_epilogue(C.ctypes.data, C.strides[0], capi.F32, capi.STEP_BIAS, bias.ctypes.data)
    w.matmul_host(A.ctypes.data, capi.BF16, M, K, A.strides[0], ep)
    ref = port.postops(port.gemm_bf16(A, B), port.BIAS, port.F32, bias=bias)
    assert H.rel_to_max(C, ref) < 1e-5


def test_argument_errors():
    rng = np.random.default_rng(1)
    B = H.two_valued_bf16(rng, (64, 64))
    w = H.pack(B)
    A = H.Dev(H.two_valued_bf16(rng, (4, 64)))
    C = H.Dev(shape=(4, 64), dtype=np.float32)
    ep = capi.make_epilogue(C.ptr, C.ld, capi.F32)
    with pytest.raises(capi.B200FCError) as e:
        w.matmul(A.ptr, capi.BF16, 4, 32, 128, ep)      # K mismatch
    assert e.value.code == capi.ERR_INVALID
    with pytest.raises(capi.B200FCError):
        w.matmul(A.ptr, capi.S8, 4, 64, 128, ep)        # dtype mismatch
    with pytest.raises(capi.B200FCError):
        w.matmul(A.ptr, capi.BF16, 4, 64, 128, ep, 0, 65)   # n1 > N
    ep2 = capi.make_epilogue(C.ptr, C.ld, capi.F32, capi.STEP_BIAS)  # bias missing
    with pytest.raises(capi.B200FCError):
        w.matmul(A.ptr, capi.BF16, 4, 64, 128, ep2)


def test_decode_ctas_per_sm_setter():
    """one CTA per SM (for independent layers on several streams) computes the same values as the default two"""
    rng = np.random.default_rng(21)
    M, K, N = 4, 4096, 1536
    x = H.normal_bf16(rng, (M, K))
    Wq = rng.integers(-127, 128, (K, N), dtype=np.int8)
    scale = rng.uniform(0.001, 0.02, N).astype(np.float32)
    w = H.pack(Wq, False, capi.PACK_INT8_CHANNEL, scales=scale)
    ref = port.postops(port.gemm_bf16_w8(x, Wq), port.DEQUANT, port.F32, deq_scale=1.0, deq_scale_per_oc=scale)
    try:
        capi.set_decode_ctas_per_sm(1)
        got1 = H.run_matmul(w, x, capi.F32, steps=capi.STEP_DEQUANT)
    finally:
        capi.set_decode_ctas_per_sm(0)
    got2 = H.run_matmul(w, x, capi.F32, steps=capi.STEP_DEQUANT)
    assert H.rel_to_max(got1, ref) < 1e-5 and H.rel_to_max(got2, ref) < 1e-5
    with pytest.raises(capi.B200FCError):
        capi.set_decode_ctas_per_sm(3)


def test_tensor_memory_decode_kernel_all_row_counts_subprocess():
    """The decode kernel on the tcgen05 tensor cores takes calls with more than 8 rows by default; B200FC_GEMV_TC=2 (read
    once per process, hence the child) routes every decode-shaped bf16 call through it: M = 1..16, K and N tails, a column
    range, bias + GeLU, exact on two-valued data."""
    import os, subprocess, sys, textwrap
    code = textwrap.dedent("""
        import numpy as np
        import helpers as H
        from mm_amx_b200 import capi
        from oracle import port
        rng = np.random.default_rng(3)
        for (M, K, N) in [(1, 4096, 4096), (3, 1000, 777), (8, 2560, 10752), (11, 320, 257), (16, 8192, 1536)]:
            A = H.two_valued_bf16(rng, (M, K)); B = H.two_valued_bf16(rng, (K, N))
            w = H.pack(B)
            got = H.run_matmul(w, A, capi.F32)
            assert np.array_equal(got, port.gemm_bf16(A, B)), (M, K, N)
        M, K, N = 5, 1536, 1000
        A = H.normal_bf16(rng, (M, K)); B = H.normal_bf16(rng, (N, K), 0.02)
        bias = rng.standard_normal(N).astype(np.float32)
        w = H.pack(B, True)
        got = H.run_matmul(w, A, capi.F32, steps=capi.STEP_BIAS | capi.STEP_GELU, bias=bias, n0=128, n1=900)
        ref = port.postops(port.gemm_bf16(A, B, transposeB=True), port.BIAS | port.GELU, port.F32, bias=bias)
        assert H.rel_to_max(got[:, 128:900], ref[:, 128:900]) < 1e-5
        assert (np.delete(got, np.s_[128:900], axis=1).view(np.uint32) == 0xCDCDCDCD).all()
        print("tc ok")
    """)
    env = dict(os.environ, B200FC_GEMV_TC="2")
    here = os.path.dirname(os.path.abspath(__file__))
    env["PYTHONPATH"] = os.pathsep.join([here, os.path.dirname(here), env.get("PYTHONPATH", "")])
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "tc ok" in r.stdout, r.stdout + r.stderr
