"""Debug bounds checks of the matmul epilogues (the stand-in for a memory checker on this path): with the switch on,
every store address computed by hand from tile coordinates is compared with the extent of C. Clean runs stay clean; a
test-only shrink of the extent makes the check fire, the store is skipped (nothing outside memory is touched) and the
status call reports it."""
import ctypes as C

import numpy as np
import pytest

from beantensor_b200 import _lib, sharding
from beantensor_b200.errors import CudaError, DeviceTimeout
from tests.helpers import TOL, gemm_inputs, to_gpu, to_host_bits, torch_dtype

pytestmark = pytest.mark.gpu


@pytest.fixture
def bounds():
    L = _lib.lib()
    assert L.btm_debug_set(b"bounds", 1) == _lib.OK
    yield L
    assert L.btm_debug_set(b"bounds_shrink", 0) == _lib.OK
    assert L.btm_debug_set(b"bounds", 0) == _lib.OK


@pytest.mark.parametrize("dtype", [_lib.F16, _lib.F32])
def test_clean_runs_stay_clean(btm, oracle, bounds, dtype):
    import torch
    # per-thread row stores (output pitch not a multiple of 16 bytes) and the TMA-store path, ragged shapes
    for (M, N, K, pad) in [(129, 65, 72, 3), (257, 130, 136, 1), (300, 520, 200, 0)]:
        A, B = gemm_inputs(dtype, M, N, K, 5 + M, "uniform" if dtype == _lib.F32 else "normal")
        big = torch.full((M, N + pad), float("nan"), dtype=torch_dtype(dtype), device="cuda")
        out = big[:, :N]
        btm.matmul_gpu(to_gpu(A, dtype), to_gpu(B, dtype), out)
        btm.check_device_status(0)
        assert oracle.rel_frobenius(to_host_bits(out, dtype), dtype, oracle.gemm(dtype, A, B)) <= TOL[dtype]


def test_peer_stores_of_the_sharded_product_stay_inside(btm, oracle, bounds):
    import torch
    dtype, world, (M, N, K) = _lib.BF16, 8, (300, 2048, 128)
    A, B = gemm_inputs(dtype, M, N, K, 21)
    a, b = to_gpu(A, dtype), to_gpu(B, dtype)
    copies = [torch.full((M, N), float("nan"), dtype=torch_dtype(dtype), device="cuda") for _ in range(world)]
    table = (C.c_void_p * world)(*[c.data_ptr() for c in copies])
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for r in range(world):
        c0, c1 = sharding.column_block(N, r, world)
        b_loc = b[:, c0:c1].contiguous()
        assert bounds.btm_gemm_nshard(0, st, dtype, M, c1 - c0, K, a.data_ptr(), K, b_loc.data_ptr(), c1 - c0, table, N, r, world) == _lib.OK
    btm.check_device_status(0)
    ref = oracle.gemm(dtype, A, B)
    for c in copies:
        assert oracle.rel_frobenius(to_host_bits(c, dtype), dtype, ref) <= TOL[dtype]


def test_a_store_past_the_extent_is_skipped_and_reported(btm, oracle, bounds):
    import torch
    dtype, (M, N, K) = _lib.F16, (130, 72, 64)   # operands fit the tensor-core kernel, the output pitch (75) does not:
    A, B = gemm_inputs(dtype, M, N, K, 9)        # per-thread row stores, the path whose addresses are computed by hand
    big = torch.full((M, N + 3), float("nan"), dtype=torch.float16, device="cuda")
    out = big[:, :N]
    assert bounds.btm_debug_set(b"bounds_shrink", 5) == _lib.OK   # pretend the last 5 elements are not ours
    btm.matmul_gpu(to_gpu(A, dtype), to_gpu(B, dtype), out)
    with pytest.raises(CudaError) as e:
        btm.check_device_status(0)
    assert not isinstance(e.value, DeviceTimeout) and "bounds" in str(e.value)
    btm.check_device_status(0)                                    # reported once
    assert torch.isnan(out[M - 1, N - 5:]).all()                  # the offending store was not made ...
    ref = oracle.gemm(dtype, A, B)
    got = to_host_bits(out, dtype)
    assert oracle.rel_frobenius(got[:-1], dtype, ref[:-1]) <= TOL[dtype]   # ... and every other row is complete and right
    assert bounds.btm_debug_set(b"bounds_shrink", 0) == _lib.OK
    btm.matmul_gpu(to_gpu(A, dtype), to_gpu(B, dtype), out)
    btm.check_device_status(0)
    assert oracle.rel_frobenius(to_host_bits(out, dtype), dtype, ref) <= TOL[dtype]
