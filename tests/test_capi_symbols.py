"""CPU: the C-ABI library loads, exports every function include/b200fc.h declares, and the Python binding lists the
same set.  No compute call is made (there is no GPU here)."""
import ctypes
import os
import re

import pytest

from mm_amx_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    src = open(os.path.join(ROOT, "include", "b200fc.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    names = re.findall(r"\b(b200fc_[a-z0-9_]+)\s*\(", src)
    return sorted(set(names))


def test_library_builds_and_loads():
    from mm_amx_b200 import build
    path = build.build_library()
    assert os.path.exists(path)
    assert capi.lib().b200fc_version().startswith(b"b200fc")


def test_every_declared_symbol_is_exported_and_bound():
    L = ctypes.CDLL(capi.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(L, n), "missing export " + n
    assert sorted(capi.SIGNATURES) == names


def test_epilogue_struct_layout_matches_header():
    # int, int, void*, int64, const float*, float, const float*, float, const float*
    assert ctypes.sizeof(capi.Epilogue) == 64
    assert capi.Epilogue.C.offset == 8 and capi.Epilogue.ldc_bytes.offset == 16
    assert capi.Epilogue.deq_scale.offset == 32 and capi.Epilogue.deq_scale_per_oc.offset == 40
    assert capi.Epilogue.q_scale.offset == 48 and capi.Epilogue.q_scale_per_oc.offset == 56


def test_allreduce_struct_layout_matches_header(tmp_path):
    """compile the header with the host C compiler and compare sizeof / offsetof with the ctypes mirror"""
    import subprocess
    src = tmp_path / "layout.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "b200fc.h"\n'
        'int main(void) { printf("%zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(b200fc_allreduce_t),\n'
        '  offsetof(b200fc_allreduce_t, partial_local), offsetof(b200fc_allreduce_t, partial_mc),\n'
        '  offsetof(b200fc_allreduce_t, out_mc), offsetof(b200fc_allreduce_t, ld_bytes),\n'
        '  offsetof(b200fc_allreduce_t, flags), offsetof(b200fc_allreduce_t, max_tiles),\n'
        '  offsetof(b200fc_allreduce_t, comm_sms)); return 0; }\n')
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    got = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    A = capi.AllReduce
    assert got == [ctypes.sizeof(A), A.partial_local.offset, A.partial_mc.offset, A.out_mc.offset, A.ld_bytes.offset,
                   A.flags.offset, A.max_tiles.offset, A.comm_sms.offset]


def test_allreduce_argument_checks_need_no_gpu():
    L = capi.lib()
    rc = L.b200fc_mlp_down_allreduce(None, 64, None, None)
    assert rc == capi.ERR_INVALID and b"null" in L.b200fc_last_error()


def test_weight_import_rejects_foreign_blobs_without_gpu():
    L = capi.lib()
    h = ctypes.c_void_p()
    for raw in (b"", b"short", b"x" * 64, b"B2FCWGT1" + b"\0" * 56, b"B2FCWGT1" + (64).to_bytes(4, "little") + b"\xff" * 52):
        buf = ctypes.create_string_buffer(raw, max(len(raw), 1))
        rc = L.b200fc_weight_import(buf, len(raw), ctypes.byref(h), None)
        assert rc == capi.ERR_INVALID, raw[:12]
    assert L.b200fc_weight_import(None, 64, ctypes.byref(h), None) == capi.ERR_INVALID
    n = ctypes.c_size_t()
    assert L.b200fc_weight_export_size(None, ctypes.byref(n)) == capi.ERR_INVALID


def test_argument_checks_need_no_gpu():
    L = capi.lib()
    h = ctypes.c_void_p()
    rc = L.b200fc_weight_pack(None, capi.BF16, 64, 64, 128, 0, 0, None, ctypes.byref(h), None)
    assert rc == capi.ERR_INVALID and b"null" in L.b200fc_last_error()
    buf = (ctypes.c_char * 64)()
    rc = L.b200fc_weight_pack(buf, capi.F32, 4, 4, 16, 0, 0, None, ctypes.byref(h), None)
    assert rc == capi.ERR_INVALID
    rc = L.b200fc_mlp_create(buf, buf, buf, 100, 64, 0, 1, ctypes.byref(h), None)   # K % 64 != 0
    assert rc == capi.ERR_INVALID
    rc = L.b200fc_mlp_create(buf, buf, buf, 64, 96, 0, 2, ctypes.byref(h), None)    # (N / tp) % 32 != 0
    assert rc == capi.ERR_INVALID
    with pytest.raises(capi.B200FCError):
        capi.check(rc)


def test_reference_module_name_is_importable():
    """a script written against the reference's extension does `import amx_mlp` (torch-ext/setup.py:10-13)"""
    import importlib
    m = importlib.import_module("amx_mlp")
    from mm_amx_b200 import amx_mlp as inner
    assert m.LinearNxN is inner.LinearNxN and m.MLP is inner.MLP and m.clflush is inner.clflush
