"""The C++23 binding above the C ABI compiles with the host toolchain and keeps the reference's
error convention. No GPU: only guards and status mapping run."""
import os
import shutil
import subprocess

import pytest

from beantensor_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_binding_compiles_and_maps_errors(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    _lib.lib()
    exe = tmp_path / "host_binding"
    libdir = os.path.join(ROOT, "beantensor_b200")
    cmd = [gxx, "-std=c++23", "-O1", "-Wall", os.path.join(ROOT, "tests", "host_binding_main.cpp"), "-o", str(exe),
           f"-L{libdir}", "-lbtm", f"-Wl,-rpath,{libdir}"]
    subprocess.check_call(cmd)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "passed=6" in r.stdout
