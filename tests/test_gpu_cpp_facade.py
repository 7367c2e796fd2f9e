"""GPU: builds and runs the C++ accuracy program for the header-only façade (include/mm_amx_gpu.hpp), which mirrors
the reference's own main()-style checks (see tests/cpp/test_facade.cpp)."""
import os
import subprocess

import pytest

from mm_amx_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_program(out):
    libdir = os.path.dirname(capi.LIB_PATH)
    cmd = ["/usr/bin/g++", "-O1", "-std=c++14", "-I" + os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "test_facade.cpp"), "-L" + libdir, "-lb200fc",
           "-Wl,-rpath," + libdir, "-o", out]
    subprocess.check_call(cmd)


def test_facade_header_compiles(tmp_path):
    """CPU: the façade is plain C++14 and links against the C ABI."""
    capi.lib()
    build_program(str(tmp_path / "test_facade"))


@pytest.mark.gpu
def test_facade_accuracy_program(tmp_path):
    exe = str(tmp_path / "test_facade")
    build_program(exe)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    tail = "\n".join(r.stdout.splitlines()[-25:])
    assert r.returncode == 0, tail + r.stderr[-2000:]
    assert "PASS: 0 failure(s)" in r.stdout
    assert r.stdout.count("Match") >= 150
