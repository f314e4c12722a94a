"""Fused bias + ReLU epilogue (btm_gemm_bias_act) against the fp64 oracle.

out = relu(A.B + bias), bias and activation applied to the fp32 accumulator before the one rounding to the
output type. Covers the two tensor-core kernels, the fp32 (3xTF32) path and the general CUDA-core kernel."""
import numpy as np
import pytest

from beantensor_b200 import _lib, synth
from tests.helpers import TOL, gemm_inputs, store, to_gpu, to_host_bits, torch_dtype

pytestmark = pytest.mark.gpu


def _reference(oracle, dtype, A, B, bias_bits, relu):
    ref = oracle.gemm(dtype, A, B)
    if bias_bits is not None:
        ref = ref + oracle.widen(bias_bits, dtype)[None, :]
    if relu:
        ref = np.maximum(ref, 0.0)
    return ref


@pytest.mark.parametrize("dtype", [_lib.F16, _lib.BF16, _lib.F32])
@pytest.mark.parametrize("shape", [(256, 512, 128), (130, 72, 96), (129, 75, 33), (1, 8, 8), (300, 1024, 64)])
@pytest.mark.parametrize("use_bias,relu", [(True, False), (False, True), (True, True)])
def test_bias_relu_matches_oracle(btm, oracle, dtype, shape, use_bias, relu):
    import torch
    M, N, K = shape
    A, B = gemm_inputs(dtype, M, N, K, 31)
    bias_bits = store(synth.normal((N,), 0.5, 31, 2), dtype) if use_bias else None
    a, b = to_gpu(A, dtype), to_gpu(B, dtype)
    bias = to_gpu(bias_bits, dtype) if use_bias else None
    out = torch.full((M, N), float("nan"), dtype=torch_dtype(dtype), device="cuda")
    btm.matmul_gpu(a, b, out, bias=bias, relu=relu)
    btm.check_device_status(0)
    got = to_host_bits(out, dtype)
    ref = _reference(oracle, dtype, A, B, bias_bits, relu)
    assert oracle.rel_frobenius(got, dtype, ref) <= TOL[dtype]
    if relu:
        assert float(out.float().min()) >= 0.0


@pytest.mark.parametrize("kernel", ["1cta", "2cta"])
def test_both_tensor_core_kernels(btm, oracle, kernel, monkeypatch):
    import torch
    monkeypatch.setenv("BTM_FORCE_KERNEL", kernel)
    dtype, (M, N, K) = _lib.F16, (512, 768, 512)
    A, B = gemm_inputs(dtype, M, N, K, 32)
    bias_bits = store(synth.normal((N,), 0.5, 32, 2), dtype)
    out = torch.empty((M, N), dtype=torch.float16, device="cuda")
    btm.matmul_gpu(to_gpu(A, dtype), to_gpu(B, dtype), out, bias=to_gpu(bias_bits, dtype), relu=True)
    ref = _reference(oracle, dtype, A, B, bias_bits, True)
    assert oracle.rel_frobenius(to_host_bits(out, dtype), dtype, ref) <= TOL[dtype]


def test_no_bias_no_activation_is_the_plain_product(btm):
    import torch
    dtype, (M, N, K) = _lib.BF16, (256, 256, 256)
    A, B = gemm_inputs(dtype, M, N, K, 33)
    a, b = to_gpu(A, dtype), to_gpu(B, dtype)
    plain = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    fused = torch.empty_like(plain)
    btm.matmul_gpu(a, b, plain)
    L = _lib.lib()
    import ctypes as C
    rc = L.btm_gemm_bias_act(0, C.c_void_p(torch.cuda.current_stream().cuda_stream), dtype, M, N, K, a.data_ptr(), K, b.data_ptr(), N,
                             None, 0, fused.data_ptr(), N)
    assert rc == _lib.OK
    assert torch.equal(plain, fused)


def test_bad_activation_code(btm):
    import torch
    t = torch.zeros((8, 8), dtype=torch.float16, device="cuda")
    rc = _lib.lib().btm_gemm_bias_act(0, None, _lib.F16, 8, 8, 8, t.data_ptr(), 8, t.data_ptr(), 8, None, 7, t.data_ptr(), 8)
    assert rc == _lib.ERR_INVALID
