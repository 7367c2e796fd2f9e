"""GPU parity of the fused Llama MLP and of the matrix-vector product against the CPU oracle, through the C ABI.

MLP tolerance: max|err| / max|ref| <= 1e-2 after bf16 output rounding (the reference's own test uses rtol 0.05 /
atol 0.01, tests/amx-mlp.cpp:876); on two-valued +-0.5 inputs (its test data) the result is compared much tighter.
"""
import numpy as np
import pytest

from oracle import port
from oracle._common import bf16_bits, bf16_to_f32
from mm_amx_b200 import capi
import helpers as H

pytestmark = pytest.mark.gpu


def make_mlp_inputs(rng, M, K, N, two_valued=False):
    if two_valued:
        return (H.two_valued_bf16(rng, (M, K)), H.two_valued_bf16(rng, (N, K)), H.two_valued_bf16(rng, (N, K)),
                H.two_valued_bf16(rng, (K, N)))
    return (H.normal_bf16(rng, (M, K)), H.normal_bf16(rng, (N, K), 0.02), H.normal_bf16(rng, (N, K), 0.02),
            H.normal_bf16(rng, (K, N), 0.02))


def run_mlp(x, gate, up, down, tp_rank=0, tp_size=1, partial_dtype=None, host_weights=False):
    M, K = x.shape
    N = gate.shape[0]
    if host_weights:
        mlp = capi.Mlp(gate.ctypes.data, up.ctypes.data, down.ctypes.data, K, N, tp_rank, tp_size)
    else:
        dg, du, dd = H.Dev(gate), H.Dev(up), H.Dev(down)
        mlp = capi.Mlp(dg.ptr, du.ptr, dd.ptr, K, N, tp_rank, tp_size)
    dx = H.Dev(x)
    if partial_dtype is None:
        out = H.Dev(shape=(M, K), dtype=np.uint16)
        mlp.run(dx.ptr, dx.ld, M, out.ptr, out.ld)
    else:
        out = H.Dev(shape=(M, K), dtype=H.NP_OF[partial_dtype])
        mlp.run_partial(dx.ptr, dx.ld, M, out.ptr, partial_dtype, out.ld)
    capi.sync_check()
    Ns = N // tp_size
    act = np.empty((M, Ns), np.uint16)
    capi.memcpy(act.ctypes.data, mlp.act_ptr(), act.nbytes)
    return out.numpy(), act


@pytest.mark.parametrize("M", [1, 5, 16, 17, 130, 300])
def test_mlp_random(M):
    rng = np.random.default_rng(100 + M)
    K, N = 512, 1280
    x, gate, up, down = make_mlp_inputs(rng, M, K, N)
    ref, ref_act = port.mlp(x, gate, up, down, want_act=True)
    got, act = run_mlp(x, gate, up, down)
    assert H.rel_to_max(bf16_to_f32(act), bf16_to_f32(ref_act)) < 1e-2
    assert H.rel_to_max(bf16_to_f32(got), bf16_to_f32(ref)) < 1e-2


@pytest.mark.parametrize("M", [2, 33])
def test_mlp_two_valued(M):
    """the reference's own test data (+-0.5, tests/amx-mlp.cpp:845-881): GEMM sums are exact, only SiLU differs
    (expf + division here, exp polynomial + rcp14 there), by at most 1 bf16 ulp of the activation."""
    rng = np.random.default_rng(M)
    K, N = 256, 512
    x, gate, up, down = make_mlp_inputs(rng, M, K, N, two_valued=True)
    ref, ref_act = port.mlp(x, gate, up, down, want_act=True)
    got, act = run_mlp(x, gate, up, down, host_weights=True)
    a, r = bf16_to_f32(act), bf16_to_f32(ref_act)
    assert np.abs(a - r).max() <= np.abs(r).max() * 2.0 ** -7
    assert H.rel_to_max(bf16_to_f32(got), bf16_to_f32(ref)) < 1e-2


@pytest.mark.parametrize("M", [4, 48])
@pytest.mark.parametrize("tp", [2, 4])
def test_mlp_tensor_parallel_shards(M, tp):
    """Megatron split on one GPU: the fp32 partials of all shards sum to the full result."""
    rng = np.random.default_rng(M * tp)
    K, N = 256, 1024
    x, gate, up, down = make_mlp_inputs(rng, M, K, N)
    ref = port.mlp(x, gate, up, down)
    total = np.zeros((M, K), np.float32)
    Ns = N // tp
    for r in range(tp):
        part, _ = run_mlp(x, gate, up, down, r, tp, capi.F32)
        _, _, oracle_part = port.mlp(x, gate[r * Ns:(r + 1) * Ns], up[r * Ns:(r + 1) * Ns],
                                     np.ascontiguousarray(down[:, r * Ns:(r + 1) * Ns]), want_act=True,
                                     want_partial=True)
        assert H.rel_to_max(part, oracle_part) < 2e-3
        total += part
    got = port.f32_to_bf16(total)
    assert H.rel_to_max(bf16_to_f32(got), bf16_to_f32(ref)) < 1e-2


def test_mlp_many_tiles():
    """gate/up with more tiles than CTA pairs (several rounds of the persistent schedule, SiLU pairing in each)"""
    rng = np.random.default_rng(77)
    M, K, N = 520, 128, 5312
    x, gate, up, down = make_mlp_inputs(rng, M, K, N)
    ref, ref_act = port.mlp(x, gate, up, down, want_act=True)
    got, act = run_mlp(x, gate, up, down)
    assert H.rel_to_max(bf16_to_f32(act), bf16_to_f32(ref_act)) < 1e-2
    assert H.rel_to_max(bf16_to_f32(got), bf16_to_f32(ref)) < 1e-2
    # element-wise too: a misplaced tile would leave whole column ranges wrong but small
    assert np.abs(bf16_to_f32(act) - bf16_to_f32(ref_act)).max() < 0.02 * np.abs(bf16_to_f32(ref_act)).max()


def test_mlp_long_k_few_tiles():
    """M just above the decode limit with a long K: both GEMMs take the split-K route (SiLU pairing in the reduction)"""
    rng = np.random.default_rng(77)
    M, K, N = 40, 2048, 4096
    x, gate, up, down = make_mlp_inputs(rng, M, K, N)
    ref, ref_act = port.mlp(x, gate, up, down, want_act=True)
    got, act = run_mlp(x, gate, up, down)
    assert H.rel_to_max(bf16_to_f32(act), bf16_to_f32(ref_act)) < 1e-2
    assert H.rel_to_max(bf16_to_f32(got), bf16_to_f32(ref)) < 1e-2


def test_mlp_host_entry_point():
    rng = np.random.default_rng(3)
    M, K, N = 24, 256, 512
    x, gate, up, down = make_mlp_inputs(rng, M, K, N)
    mlp = capi.Mlp(gate.ctypes.data, up.ctypes.data, down.ctypes.data, K, N)
    out = np.zeros((M, K), np.uint16)
    mlp.run_host(x.ctypes.data, x.strides[0], M, out.ctypes.data, out.strides[0])
    ref = port.mlp(x, gate, up, down)
    assert H.rel_to_max(bf16_to_f32(out), bf16_to_f32(ref)) < 1e-2


def test_mlp_ragged_last_round():
    """gate/up with 4 x 19 = 76 tiles on 74 CTA pairs and K = 6144: its two left-over tiles take the K-split route with
    the SiLU * up pairing in the reduction kernel; rows from both regions against the CPU oracle (rows are independent)"""
    rng = np.random.default_rng(19)
    M, K, N = 900, 6144, 2432
    x, gate, up, down = make_mlp_inputs(rng, M, K, N)
    got, act = run_mlp(x, gate, up, down)
    rows = np.r_[0:8, 380:388, 512:520, 760:776, 892:900]
    ref, ref_act = port.mlp(x[rows], gate, up, down, want_act=True)
    assert H.rel_to_max(bf16_to_f32(act[rows]), bf16_to_f32(ref_act)) < 1e-2
    assert H.rel_to_max(bf16_to_f32(got[rows]), bf16_to_f32(ref)) < 1e-2
    assert np.abs(bf16_to_f32(act[rows]) - bf16_to_f32(ref_act)).max() < 0.02 * np.abs(bf16_to_f32(ref_act)).max()


@pytest.mark.parametrize("M", [512, 700, 1100])
def test_mlp_host_entry_point_mid_size_batches(M):
    """from M = 512 on the host-buffer call is pipelined with the library's own choice of row chunks"""
    rng = np.random.default_rng(M)
    K, N = 256, 512
    x, gate, up, down = make_mlp_inputs(rng, M, K, N)
    mlp = capi.Mlp(gate.ctypes.data, up.ctypes.data, down.ctypes.data, K, N)
    out = np.zeros((M, K), np.uint16)
    mlp.run_host(x.ctypes.data, x.strides[0], M, out.ctypes.data, out.strides[0])
    capi.sync_check()
    assert H.rel_to_max(bf16_to_f32(out), bf16_to_f32(port.mlp(x, gate, up, down))) < 1e-2


@pytest.mark.parametrize("plan", [None, "1,3,5;4,1,1,3", "2;9", "9;1,1"])
def test_mlp_host_entry_point_large_batch_is_pipelined(plan, monkeypatch):
    """large batches go through the copy / compute / copy pipeline, gate/up and down cut into row chunks independently
    (the library's own choice, and forced uneven ones); rows must land where they belong."""
    if plan is None:
        monkeypatch.delenv("B200FC_HOST_PLAN", raising=False)
    else:
        monkeypatch.setenv("B200FC_HOST_PLAN", plan)
    rng = np.random.default_rng(4)
    M, K, N = 2300, 256, 512
    x, gate, up, down = make_mlp_inputs(rng, M, K, N)
    mlp = capi.Mlp(gate.ctypes.data, up.ctypes.data, down.ctypes.data, K, N)
    out = np.zeros((M, K + 8), np.uint16)[:, :K]          # strided host output
    xs = np.zeros((M, K + 16), np.uint16)[:, :K]; xs[:] = x  # strided host input
    for _ in range(2):                                     # the second call reuses the cached plan and the events
        out[:] = 0
        mlp.run_host(xs.ctypes.data, xs.strides[0], M, out.ctypes.data, out.strides[0])
        capi.sync_check()
        ref = port.mlp(x, gate, up, down)
        assert H.rel_to_max(bf16_to_f32(np.ascontiguousarray(out)), bf16_to_f32(ref)) < 1e-2
    dx = H.Dev(x); dout = H.Dev(shape=(M, K), dtype=np.uint16)
    mlp.run(dx.ptr, dx.ld, M, dout.ptr, dout.ld)
    capi.sync_check()
    # the same kernels row by row; a chunk of few tiles may take the split-K route, whose fp32 sums are rounded to
    # bf16 once like the others' but added in another order: at most the last bit of an element differs
    a, b = bf16_to_f32(dout.numpy()), bf16_to_f32(np.ascontiguousarray(out))
    assert np.abs(a - b).max() <= np.abs(a).max() * 2.0 ** -7
    assert (a != b).mean() < 0.02


# MatmulVector known-answer shapes: main.cpp:884-885 (M=901, K=80 / 96), test_qk.cpp:486-487 (M=256, K=128)
@pytest.mark.parametrize("M,K", [(901, 80), (901, 96), (256, 128), (64, 160), (64, 192), (7, 33), (1000, 4096)])
def test_matvec(M, K):
    rng = np.random.default_rng(M + K)
    A = H.two_valued_bf16(rng, (M, K)); b = H.two_valued_bf16(rng, (K,))
    dA, db, dc = H.Dev(A), H.Dev(b), H.Dev(shape=(M,), dtype=np.float32)
    capi.matvec(dA.ptr, capi.BF16, M, K, A.strides[0], db.ptr, dc.ptr)
    assert np.array_equal(dc.numpy(), port.matvec_bf16(A, b))
    Ai = rng.integers(-128, 128, (M, K), dtype=np.int8); bi = rng.integers(-128, 128, (K,), dtype=np.int8)
    dA, db, dc = H.Dev(Ai), H.Dev(bi), H.Dev(shape=(M,), dtype=np.int32)
    capi.matvec(dA.ptr, capi.S8, M, K, Ai.strides[0], db.ptr, dc.ptr)
    assert np.array_equal(dc.numpy(), port.matvec_s8(Ai, bi))
    c = np.zeros(M, np.float32)
    capi.matvec_host(A.ctypes.data, capi.BF16, M, K, A.strides[0], b.ctypes.data, c.ctypes.data)
    assert np.array_equal(c, port.matvec_bf16(A, b))


@pytest.mark.parametrize("M", [1, 5, 16, 40, 300])
@pytest.mark.parametrize("with_weight,residual", [(False, True), (True, False), (True, True)])
def test_rmsnorm_and_mlp_block(M, with_weight, residual):
    """RMSNorm in front of the MLP and the residual behind it (the layer step of torch-ext/test.py:161-189) against
    the oracle: the normalised activations within one bf16 ulp (rsqrt vs 1/sqrt), the block within the 1e-2 bar."""
    rng = np.random.default_rng(M * 3 + with_weight + 2 * residual)
    K, N = 512, 1280
    gate, up = H.normal_bf16(rng, (N, K), 0.02), H.normal_bf16(rng, (N, K), 0.02)
    down = H.normal_bf16(rng, (K, N), 0.02)
    x = H.normal_bf16(rng, (M, K), 1.5)
    wn = H.normal_bf16(rng, (K,), 1.0) if with_weight else None
    eps = 1e-6
    dx = H.Dev(x)
    dw = H.Dev(wn) if with_weight else None
    dn = H.Dev(shape=(M, K), dtype=np.uint16, fill=0xCD)
    capi.rmsnorm(dx.ptr, dx.ld, M, K, eps, dn.ptr, dn.ld, dw.ptr if dw else None)
    capi.sync_check()
    want_n = port.rmsnorm(x, eps, wn)
    got_n = dn.numpy()
    ulp = np.abs(got_n.astype(np.int32) - want_n.astype(np.int32))
    assert ulp.max() <= (2 if with_weight else 1), ulp.max()
    mlp = capi.Mlp(gate.ctypes.data, up.ctypes.data, down.ctypes.data, K, N)
    out = H.Dev(shape=(M, K), dtype=np.uint16, fill=0xCD)
    mlp.run_block(dx.ptr, dx.ld, M, eps, out.ptr, out.ld, dw.ptr if dw else None, residual)
    capi.sync_check()
    want = port.mlp_block(x, gate, up, down, eps, wn, residual)
    assert H.rel_to_max(bf16_to_f32(out.numpy()), bf16_to_f32(want)) < 1e-2
    # the block is the three public steps in a row: normalise, MLP, add (bit for bit when no residual is added)
    if not residual:
        plain = H.Dev(shape=(M, K), dtype=np.uint16)
        mlp.run(dn.ptr, dn.ld, M, plain.ptr, plain.ld)
        capi.sync_check()
        assert np.array_equal(plain.numpy(), out.numpy())


def test_decode_mlp_in_one_launch_subprocess():
    """B200FC_MLP_FUSED=1 (read once per process, hence the child process): gate/up and down of a decode-shaped MLP run
    as two jobs of ONE launch with a bounded grid-wide barrier between them.  Off by default (measured slower than two
    launches); the path must still be right: against the CPU oracle at M = 1, 5, 16, with and without the residual block."""
    import os, subprocess, sys, textwrap
    code = textwrap.dedent("""
        import numpy as np
        import helpers as H
        from mm_amx_b200 import capi
        from oracle import port
        from oracle._common import bf16_to_f32
        rng = np.random.default_rng(77)
        K, N = 2048, 5504
        gate = H.normal_bf16(rng, (N, K), 0.02); up = H.normal_bf16(rng, (N, K), 0.02); down = H.normal_bf16(rng, (K, N), 0.02)
        dg, du, dd = H.Dev(gate), H.Dev(up), H.Dev(down)
        mlp = capi.Mlp(dg.ptr, du.ptr, dd.ptr, K, N)
        before = capi.launch_count()
        for M in (1, 5, 16):
            x = H.normal_bf16(rng, (M, K))
            dx = H.Dev(x); out = H.Dev(shape=(M, K), dtype=np.uint16, fill=0xCD)
            n0 = capi.launch_count()
            mlp.run(dx.ptr, K * 2, M, out.ptr, K * 2)
            capi.sync_check()
            assert capi.launch_count() - n0 == 1, "expected one launch"
            ref = port.mlp(x, gate, up, down)
            assert H.rel_to_max(bf16_to_f32(out.numpy()), bf16_to_f32(ref)) < 1e-2
            out2 = H.Dev(shape=(M, K), dtype=np.uint16, fill=0xCD)
            mlp.run_block(dx.ptr, K * 2, M, 1e-5, out2.ptr, K * 2)
            capi.sync_check()
            ref2 = port.mlp_block(x, gate, up, down, 1e-5)
            assert H.rel_to_max(bf16_to_f32(out2.numpy()), bf16_to_f32(ref2)) < 1e-2
        print("fused ok")
    """)
    env = dict(os.environ, B200FC_MLP_FUSED="1")
    here = os.path.dirname(os.path.abspath(__file__))
    env["PYTHONPATH"] = os.pathsep.join([here, os.path.dirname(here), env.get("PYTHONPATH", "")])
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "fused ok" in r.stdout, r.stdout + r.stderr
