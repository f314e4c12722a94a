"""Batched matmul parity."""
import numpy as np
import pytest

from beantensor_b200 import _lib, synth
from tests.helpers import TOL, store, to_gpu, to_host_bits, torch_dtype

pytestmark = pytest.mark.gpu


def run(btm, oracle, dtype, B, M, N, K, seed):
    import torch
    std = 1.0 / np.sqrt(K)
    A = store(synth.normal((B, M, K), std, seed, 0), dtype)
    Bm = store(synth.normal((B, K, N), std, seed, 1), dtype)
    out = torch.full((B, M, N), float("nan"), dtype=torch_dtype(dtype), device="cuda")
    btm.bmm_gpu(to_gpu(A, dtype), to_gpu(Bm, dtype), out)
    btm.check_device_status(0)
    got = to_host_bits(out, dtype)
    ref = oracle.bmm(dtype, A, Bm)
    return oracle.rel_frobenius(got, dtype, ref), got, ref


def test_workload_shape_fp16(btm, oracle):
    # [64,512,128] x [64,128,512] -> [64,512,512]
    err, got, ref = run(btm, oracle, _lib.F16, 64, 512, 512, 128, 3)
    assert err <= TOL[_lib.F16]
    # every product individually, so that a swapped batch index cannot hide in the norm
    for b in (0, 1, 31, 63):
        assert oracle.rel_frobenius(got[b], _lib.F16, ref[b]) <= TOL[_lib.F16]


@pytest.mark.parametrize("dtype", [_lib.F16, _lib.BF16])
@pytest.mark.parametrize("shape", [(1, 128, 256, 64), (3, 130, 72, 40), (5, 64, 64, 64), (2, 257, 129, 136), (7, 9, 11, 13)])
def test_shapes(btm, oracle, dtype, shape):
    err, _, _ = run(btm, oracle, dtype, *shape, seed=sum(shape))
    assert err <= TOL[dtype], (shape, err)


def test_batch_strides_with_gaps(btm, oracle):
    import torch
    dtype = _lib.F16
    B, M, N, K = 4, 96, 80, 64
    std = 1.0 / np.sqrt(K)
    A = store(synth.normal((B, M, K), std, 9, 0), dtype)
    Bm = store(synth.normal((B, K, N), std, 9, 1), dtype)
    a = torch.zeros((B, M + 8, K), dtype=torch.float16, device="cuda")
    a[:, :M] = to_gpu(A, dtype)
    out = torch.empty((B, M, N), dtype=torch.float16, device="cuda")
    btm.bmm_gpu(a[:, :M], to_gpu(Bm, dtype), out)
    assert oracle.rel_frobenius(to_host_bits(out, dtype), dtype, oracle.bmm(dtype, A, Bm)) <= TOL[dtype]
