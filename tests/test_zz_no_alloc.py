"""GPU: the allocation-free decode MLP entry point (b200fc_mlp_run_decode_static) against b200fc_mlp_run.

Collected last on purpose (file name), so a run that stops at the first failure has already run everything else.
The entry point serves callers that may not allocate while they run; its activation scratch is a fixed device array
inside the library that every call shares and that keeps the previous call's contents.  So the test makes two calls
in a row with different inputs and a different M — the second call meets the leftovers of the first — and compares
each result with the ordinary entry point, which runs the same kernels on a cudaMalloc'ed buffer: the outputs must be
bit-identical.  It passes in a fresh process as well as after the other tests, because the only state involved is
the per-device address lookup, which the first call performs.
"""
import numpy as np
import pytest

from mm_amx_b200 import capi
import helpers as H

pytestmark = pytest.mark.gpu


def test_decode_static_matches_allocating_entry_point_twice():
    rng = np.random.default_rng(2026)
    K, N = 512, 1280
    gate, up = H.normal_bf16(rng, (N, K), 0.02), H.normal_bf16(rng, (N, K), 0.02)
    down = H.normal_bf16(rng, (K, N), 0.02)
    mlp = capi.Mlp(gate.ctypes.data, up.ctypes.data, down.ctypes.data, K, N)
    import torch
    for call, M in enumerate((16, 3)):      # second call: fewer rows, scratch still holds the first call's rows
        x = H.normal_bf16(rng, (M, K))
        dx = H.Dev(x)
        want = H.Dev(shape=(M, K), dtype=np.uint16)
        mlp.run(dx.ptr, dx.ld, M, want.ptr, want.ld)
        got = H.Dev(shape=(M, K), dtype=np.uint16, fill=0xCD)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]          # cudaMemGetInfo: bytes the driver could still hand out
        mlp.run_decode_static(dx.ptr, dx.ld, M, got.ptr, capi.BF16, got.ld)
        capi.sync_check()
        if call == 1:
            # the first call may make the driver load kernels; by the second nothing at all may be taken from the device
            assert torch.cuda.mem_get_info()[0] == free_before
        w, g = want.numpy(), got.numpy()
        assert np.isfinite(H.bf16_to_f32(g)).all()
        assert np.array_equal(g, w)         # same kernels, same arithmetic: tolerance zero


def test_decode_static_rejects_what_does_not_fit():
    rng = np.random.default_rng(1)
    K, N = 64, 64
    z = H.normal_bf16(rng, (N, K), 0.02)
    mlp = capi.Mlp(z.ctypes.data, z.ctypes.data, np.ascontiguousarray(z.T).ctypes.data, K, N)
    x = H.Dev(H.normal_bf16(rng, (17, K)))
    out = H.Dev(shape=(17, K), dtype=np.uint16)
    with pytest.raises(capi.B200FCError) as e:
        mlp.run_decode_static(x.ptr, x.ld, 17, out.ptr, capi.BF16, out.ld)      # M > 16
    assert e.value.code == capi.ERR_INVALID and "decode" in str(e.value)
    cap = capi.lib().b200fc_mlp_decode_static_capacity()
    assert cap == 1 << 20
    # an intermediate size whose 16-row activation exceeds the scratch: 16 * 32800 * 2 bytes > 1 MiB
    Nbig = 32800 - 32800 % 32 + 32
    zb = np.zeros((Nbig, K), np.uint16)
    big = capi.Mlp(zb.ctypes.data, zb.ctypes.data, np.zeros((K, Nbig), np.uint16).ctypes.data, K, Nbig)
    with pytest.raises(capi.B200FCError) as e:
        big.run_decode_static(x.ptr, x.ld, 16, out.ptr, capi.BF16, out.ld)
    assert e.value.code == capi.ERR_INVALID and "exceeds" in str(e.value)
    big.run_decode_static(x.ptr, x.ld, 15, out.ptr, capi.BF16, out.ld)          # 15 rows fit
    capi.sync_check()
