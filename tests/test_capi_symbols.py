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
