"""Compiles and runs the C++ drop-in header check (tests/cpp/dropin_compile_test.cpp) against librib200.so."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_dropin_header_compiles_and_behaves(tmp_path):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    cuda_inc = "/usr/local/cuda/include"
    exe = tmp_path / "dropin_test"
    lib_dir = os.path.join(ROOT, "raftinfer_b200")
    subprocess.run([cxx, "-std=c++20", "-O1", "-I", os.path.join(ROOT, "include"), "-I", cuda_inc,
                    os.path.join(ROOT, "tests", "cpp", "dropin_compile_test.cpp"), "-L", lib_dir, "-lrib200",
                    f"-Wl,-rpath,{lib_dir}", "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True)
    assert "dropin ok" in out.stdout
