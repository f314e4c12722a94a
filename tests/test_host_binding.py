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


def _reference_root():
    """The reference tree, when it is present: BTM_REFERENCE_ROOT, or a directory named `reference` beside the repository."""
    for cand in (os.environ.get("BTM_REFERENCE_ROOT"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "Helper", "Threads", "CPUThreading.h")):
            return cand
    return None


def _build_async(tmp_path, with_reference_pool):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    from oracle import oracle as O
    O.build()
    _lib.lib()
    cuda_inc = "/usr/local/cuda/include"
    cuda_lib = "/usr/local/cuda/lib64"
    if not os.path.isdir(cuda_inc):
        pytest.skip("no CUDA toolkit headers")
    exe = tmp_path / "host_async"
    libdir = os.path.join(ROOT, "beantensor_b200")
    odir = os.path.join(ROOT, "oracle")
    cmd = [gxx, "-std=c++23", "-O1", "-Wall", "-pthread", os.path.join(ROOT, "tests", "host_async_main.cpp"), "-o", str(exe),
           f"-I{cuda_inc}", f"-L{libdir}", "-lbtm", f"-Wl,-rpath,{libdir}", f"-L{odir}", "-lbtm_oracle", f"-Wl,-rpath,{odir}",
           f"-L{cuda_lib}", "-lcudart", f"-Wl,-rpath,{cuda_lib}"]
    ref = _reference_root() if with_reference_pool else None
    if ref:
        cmd += ["-DBT_HAVE_REFERENCE_POOL", f"-I{ref}"]
    subprocess.check_call(cmd)
    return exe, bool(ref)


def test_async_operators_on_a_thread_pool(tmp_path):
    # With the reference tree at hand the workers run on the reference's own ThreadPool; elsewhere on a stand-in with
    # the same submit() signature. Exceptions raised in a worker surface at future.get().
    exe, used_ref = _build_async(tmp_path, with_reference_pool=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "passed=4" in r.stdout
    assert ("reference ThreadPool" in r.stdout) == used_ref


@pytest.mark.gpu
def test_async_operators_run_real_products(tmp_path):
    exe, _ = _build_async(tmp_path, with_reference_pool=True)
    r = subprocess.run([str(exe), "gpu"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "passed=6" in r.stdout
