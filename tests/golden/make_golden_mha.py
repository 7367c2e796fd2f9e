"""Generates tests/golden/golden_mha_v1.npz from the reference's own one-token attention (oracle/_ref/libmha_ref.so,
built from include/kernels_mha.hpp of the reference by `make -C oracle _ref`).  Needs the reference tree and an
AVX-512 CPU; the committed .npz travels instead.

    python tests/golden/make_golden_mha.py

Every case stores the reference OUTPUT only; the tests regenerate the seeded inputs (tests/golden_cases.py)."""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle._common import bf16_to_f32  # noqa: E402
import golden_cases as gc  # noqa: E402


def main():
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libmha_ref.so"))
    fp = ctypes.POINTER(ctypes.c_float)
    lib.ref_mha_decode.argtypes = [fp, fp, fp, fp] + [ctypes.c_int] * 5
    out = {}
    for name, c in gc.mha_cases().items():
        inp = gc.mha_inputs(c)
        B, H, N, K = c["B"], c["H"], c["N"], c["K"]
        q = np.ascontiguousarray(bf16_to_f32(inp["q"]).reshape(B, 1, H, K))
        k = np.ascontiguousarray(bf16_to_f32(inp["k"]))
        v = np.ascontiguousarray(bf16_to_f32(inp["v"]))
        o = np.zeros((B, 1, H, K), np.float32)
        rc = lib.ref_mha_decode(q.ctypes.data_as(fp), k.ctypes.data_as(fp), v.ctypes.data_as(fp), o.ctypes.data_as(fp),
                                B, H, N, K, c["bn"])
        assert rc == 0
        out[name] = o.reshape(B, H, K)
    path = os.path.join(ROOT, "tests", "golden", "golden_mha_v1.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, len(out), "cases", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
