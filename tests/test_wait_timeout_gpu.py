"""A bounded kernel wait that is made to run out: the kernel returns, the device status word holds the
wait's code, btm_check_device_status reports it once as a timeout (DeviceTimeout on the Python side), and
the device serves the next product correctly. Nothing faults and nothing hangs: the producer warps are told
to issue no loads (a flag that nothing sets from the consumers' point of view) and the consumers' waits give
up after a short limit."""
import numpy as np
import pytest

from beantensor_b200 import _lib
from beantensor_b200.errors import DeviceTimeout
from tests.helpers import TOL, gemm_inputs, to_gpu, to_host_bits

pytestmark = pytest.mark.gpu


@pytest.fixture
def hooks():
    L = _lib.lib()
    yield L
    assert L.btm_debug_set(b"skip_loads", 0) == _lib.OK
    assert L.btm_debug_set(b"wait_limit_cycles", 0) == _lib.OK


@pytest.mark.parametrize("kernel,dtype,shape", [("1cta", _lib.F16, (256, 512, 256)), ("2cta", _lib.BF16, (512, 512, 512)),
                                                ("1cta", _lib.F32, (256, 256, 128))])
def test_wait_runs_out_and_the_device_stays_usable(btm, oracle, hooks, monkeypatch, kernel, dtype, shape):
    import torch
    from tests.helpers import torch_dtype
    monkeypatch.setenv("BTM_FORCE_KERNEL", kernel)
    M, N, K = shape
    A, B = gemm_inputs(dtype, M, N, K, 77, "uniform" if dtype == _lib.F32 else "normal")
    a, b = to_gpu(A, dtype), to_gpu(B, dtype)
    out = torch.zeros((M, N), dtype=torch_dtype(dtype), device="cuda")
    btm.check_device_status(0)  # clean before the experiment

    assert hooks.btm_debug_set(b"wait_limit_cycles", 200_000) == _lib.OK  # about 0.1 ms
    assert hooks.btm_debug_set(b"skip_loads", 1) == _lib.OK
    btm.matmul_gpu(a, b, out)      # enqueues; the kernel gives up on its own
    torch.cuda.synchronize()       # returns: nothing is stuck
    with pytest.raises(DeviceTimeout):
        btm.check_device_status(0)
    btm.check_device_status(0)     # reported once, then clear

    assert hooks.btm_debug_set(b"skip_loads", 0) == _lib.OK
    assert hooks.btm_debug_set(b"wait_limit_cycles", 0) == _lib.OK
    btm.matmul_gpu(a, b, out)
    btm.check_device_status(0)
    assert oracle.rel_frobenius(to_host_bits(out, dtype), dtype, oracle.gemm(dtype, A, B)) <= TOL[dtype]


def test_unknown_switch_is_refused():
    L = _lib.lib()
    assert L.btm_debug_set(b"no_such_switch", 1) == _lib.ERR_INVALID
    assert L.btm_debug_set(None, 1) == _lib.ERR_INVALID
