"""btm_gemm_f32_static: the fp32 product for hosts that may not allocate device memory at call
time (a pool worker running while another thread holds the allocator, a process that handed all
memory to its own pool, a fixed audited budget). It keeps its scratch in a fixed array inside the
library instead of cudaMalloc'ing it, so its results must equal those of the ordinary entry point,
call after call, although every call reuses the same scratch. Collected last on purpose (file
name), so that a run that stops at the first failure has already run every other test."""
import ctypes as C

import numpy as np
import pytest

from beantensor_b200 import _lib, synth

TOL = 1e-5  # relative Frobenius error, the fp32 tolerance of the other parity tests


def _call_static(L, a, b, out):
    import torch
    M, K = a.shape
    N = b.shape[1]
    return L.btm_gemm_f32_static(0, C.c_void_p(torch.cuda.current_stream().cuda_stream), M, N, K, a.data_ptr(), a.stride(0),
                                 b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0))


def _call_ordinary(L, a, b, out):
    import torch
    M, K = a.shape
    N = b.shape[1]
    return L.btm_gemm(0, C.c_void_p(torch.cuda.current_stream().cuda_stream), _lib.F32, M, N, K, a.data_ptr(), a.stride(0),
                      b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0))


@pytest.mark.gpu
def test_two_calls_in_a_row_match_the_allocating_entry_point():
    import torch
    L = _lib.lib()
    # Two different shapes back to back: the second call finds the first call's planes in the shared
    # scratch (and a different pitch), which must not leak into its result.
    for seed, (M, N, K) in enumerate([(515, 300, 77), (256, 384, 1024)]):
        a = torch.from_numpy(synth.uniform((M, K), -1, 1, seed, 0).astype(np.float32)).cuda()
        b = torch.from_numpy(synth.uniform((K, N), -1, 1, seed, 1).astype(np.float32)).cuda()
        got = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        want = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        assert _call_static(L, a, b, got) == _lib.OK, _lib.last_error()
        assert _call_ordinary(L, a, b, want) == _lib.OK, _lib.last_error()
        torch.cuda.synchronize()
        assert not torch.isnan(got).any()
        err = ((got.double() - want.double()).norm() / want.double().norm()).item()
        assert err <= TOL, (M, N, K, err)
        # and against fp64 arithmetic directly, so that both being wrong together cannot pass
        ref = a.double() @ b.double()
        assert ((got.double() - ref).norm() / ref.norm()).item() <= TOL


@pytest.mark.gpu
def test_same_inputs_twice_give_the_same_bits():
    import torch
    L = _lib.lib()
    a = torch.from_numpy(synth.uniform((128, 96), -1, 1, 9, 0).astype(np.float32)).cuda()
    b = torch.from_numpy(synth.uniform((96, 160), -1, 1, 9, 1).astype(np.float32)).cuda()
    o1 = torch.empty((128, 160), dtype=torch.float32, device="cuda")
    o2 = torch.empty((128, 160), dtype=torch.float32, device="cuda")
    assert _call_static(L, a, b, o1) == _lib.OK, _lib.last_error()
    assert _call_static(L, a, b, o2) == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()
    assert torch.equal(o1, o2)


@pytest.mark.gpu
def test_zero_k_and_padded_rows():
    import torch
    L = _lib.lib()
    # K = 0: the product is all zeros, whatever the output held before
    a = torch.empty((5, 0), dtype=torch.float32, device="cuda")
    b = torch.empty((0, 7), dtype=torch.float32, device="cuda")
    out = torch.full((5, 7), float("nan"), dtype=torch.float32, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.btm_gemm_f32_static(0, st, 5, 7, 0, a.data_ptr(), 1, b.data_ptr(), 7, out.data_ptr(), 7) == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()
    assert torch.equal(out, torch.zeros_like(out))
    # operands that are views of wider matrices (lda > K, ldb > N, ldc > N), output pitch not a multiple of 16 bytes
    M, N, K = 130, 67, 50
    big_a = torch.from_numpy(synth.uniform((M, K + 14), -1, 1, 3, 0).astype(np.float32)).cuda()
    big_b = torch.from_numpy(synth.uniform((K, N + 5), -1, 1, 3, 1).astype(np.float32)).cuda()
    big_c = torch.full((M, N + 2), float("nan"), dtype=torch.float32, device="cuda")
    a, b, got = big_a[:, :K], big_b[:, :N], big_c[:, :N]
    assert _call_static(L, a, b, got) == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()
    ref = a.double() @ b.double()
    assert ((got.double() - ref).norm() / ref.norm()).item() <= TOL
    assert torch.isnan(big_c[:, N:]).all()  # nothing written past the N columns


def test_products_beyond_the_fixed_scratch_are_refused_with_a_clear_message():
    # Argument checks come before any device work, so this needs no GPU.
    L = _lib.lib()
    p = C.c_void_p(256)
    rc = L.btm_gemm_f32_static(0, None, 4096, 4096, 4096, p, 4096, p, 4096, p, 4096)
    assert rc == _lib.ERR_UNSUPPORTED
    msg = _lib.last_error()
    assert "scratch" in msg and "btm_gemm_f32_ws" in msg
