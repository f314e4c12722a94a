"""Parity of the dense matmul (btm_gemm through the operator mirror) with the CPU oracle."""
import numpy as np
import pytest

from beantensor_b200 import _lib
from tests.helpers import TOL, gemm_inputs, to_gpu, to_host_bits, torch_dtype

pytestmark = pytest.mark.gpu

EDGE = [1, 7, 8, 64, 65, 127, 128, 129, 257]


def run_case(btm, oracle, dtype, M, N, K, seed=11, dist="normal"):
    import torch
    A, B = gemm_inputs(dtype, M, N, K, seed, dist)
    a, b = to_gpu(A, dtype), to_gpu(B, dtype)
    out = torch.full((M, N), float("nan"), dtype=torch_dtype(dtype), device="cuda")
    btm.matmul_gpu(a, b, out)
    btm.check_device_status(0)
    got = to_host_bits(out, dtype)
    ref = oracle.gemm(dtype, A, B)
    err = oracle.rel_frobenius(got, dtype, ref)
    return err, got, ref


@pytest.mark.parametrize("dtype", [_lib.F16, _lib.BF16, _lib.F32])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 512), (384, 640, 1024), (1000, 1000, 992), (130, 72, 40)])
def test_aligned_shapes(btm, oracle, dtype, shape):
    err, _, _ = run_case(btm, oracle, dtype, *shape)
    assert err <= TOL[dtype], (shape, err)


@pytest.mark.parametrize("dtype", [_lib.F16, _lib.BF16, _lib.F32])
def test_edge_shapes(btm, oracle, dtype):
    # Every combination on the diagonal plus mixed triples: covers the tensor-core path with
    # ragged tiles, and the general kernel where the row pitch is not a multiple of 16 bytes.
    triples = [(m, m, m) for m in EDGE] + [(1, 257, 64), (257, 1, 128), (129, 65, 7), (8, 264, 72), (64, 8, 1)]
    for (M, N, K) in triples:
        err, _, _ = run_case(btm, oracle, dtype, M, N, K, seed=M * 3 + N * 5 + K)
        assert err <= TOL[dtype], ((M, N, K), err)


def test_reference_workload_fp32_1024(btm, oracle):
    # fp32, M=N=K=1024, U[-1,1] (the reference's CPU-runnable workload shape).
    err, _, _ = run_case(btm, oracle, _lib.F32, 1024, 1024, 1024, seed=0, dist="uniform")
    assert err <= 1e-5, err


def test_reference_workload_fp32_with_reference_rng(btm, oracle):
    # Same workload with A and B drawn by the restated reference generator (Tensor::random(-1,1,0)).
    import torch
    A = oracle.ref_random_f32((512, 512), 0, -1.0, 1.0, 8)
    B = oracle.ref_random_f32((512, 512), 1, -1.0, 1.0, 8)
    out = torch.empty((512, 512), dtype=torch.float32, device="cuda")
    btm.matmul_gpu(torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), out)
    assert oracle.rel_frobenius(out.cpu().numpy(), _lib.F32, oracle.gemm(_lib.F32, A, B)) <= 1e-5


def test_zero_k_and_empty(btm, oracle):
    import torch
    a = torch.empty((5, 0), dtype=torch.float16, device="cuda")
    b = torch.empty((0, 3), dtype=torch.float16, device="cuda")
    out = torch.full((5, 3), 7.0, dtype=torch.float16, device="cuda")
    btm.matmul_gpu(a, b, out)
    assert torch.count_nonzero(out).item() == 0
    out0 = torch.empty((0, 3), dtype=torch.float16, device="cuda")
    btm.matmul_gpu(torch.empty((0, 4), dtype=torch.float16, device="cuda"), torch.empty((4, 3), dtype=torch.float16, device="cuda"), out0)


def test_strided_operands_and_untouched_padding(btm, oracle):
    # lda/ldb/ldc larger than the logical width; columns beyond N must stay untouched.
    import torch
    dtype = _lib.F16
    M, N, K = 200, 136, 96
    A, B = gemm_inputs(dtype, M, N, K, 3)
    a_full = torch.zeros((M, K + 8), dtype=torch.float16, device="cuda")
    b_full = torch.zeros((K, N + 16), dtype=torch.float16, device="cuda")
    c_full = torch.full((M, N + 24), -5.0, dtype=torch.float16, device="cuda")
    a_full[:, :K] = to_gpu(A, dtype)
    b_full[:, :N] = to_gpu(B, dtype)
    btm.matmul_gpu(a_full[:, :K], b_full[:, :N], c_full[:, :N])
    got = to_host_bits(c_full[:, :N].contiguous(), dtype)
    assert oracle.rel_frobenius(got, dtype, oracle.gemm(dtype, A, B)) <= TOL[dtype]
    assert torch.all(c_full[:, N:] == -5.0)


def test_errors_follow_reference_convention(btm):
    import torch
    from beantensor_b200.errors import NotImplementedOp
    a = torch.zeros((4, 4), dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        btm.matmul_gpu(a, torch.zeros((5, 4), dtype=torch.float16, device="cuda"), a.clone())
    with pytest.raises(NotImplementedOp):
        i = torch.zeros((4, 4), dtype=torch.int32, device="cuda")
        btm.matmul_gpu(i, i, i.clone())
    with pytest.raises(ValueError):
        btm.matmul_gpu(a.cpu(), a, a.clone())


@pytest.mark.parametrize("dtype", [_lib.F16, _lib.BF16])
def test_full_size_properties(btm, oracle, dtype):
    # 4096^3 is beyond what the CPU oracle finishes in seconds, so check size-independent
    # properties: (1) sampled rows against the oracle, (2) linearity in A, (3) column-sum identity
    # 1^T (A B) = (1^T A) B evaluated in fp64.
    import torch
    M = N = K = 4096
    A, B = gemm_inputs(dtype, M, N, K, 1)
    a, b = to_gpu(A, dtype), to_gpu(B, dtype)
    out = torch.empty((M, N), dtype=torch_dtype(dtype), device="cuda")
    btm.matmul_gpu(a, b, out)
    btm.check_device_status(0)
    rows = np.array([0, 1, 127, 128, 2047, 2048, 3000, 4095])
    ref_rows = oracle.gemm(dtype, np.ascontiguousarray(A[rows]), B)
    got_rows = to_host_bits(out[torch.from_numpy(rows).cuda()], dtype)
    assert oracle.rel_frobenius(got_rows, dtype, ref_rows) <= TOL[dtype]
    # checksum of checksums
    colsum_gpu = out.double().sum(dim=0).cpu().numpy()
    colsum_ref = (oracle.widen(A, dtype).sum(axis=0)[None, :] @ oracle.widen(B, dtype)).ravel()
    assert np.linalg.norm(colsum_gpu - colsum_ref) / np.linalg.norm(colsum_ref) <= TOL[dtype]
    # linearity: (2A) B == 2 (A B) bit for bit wherever the result is a normal number (scaling by 2
    # is exact in binary floating point; in the subnormal range of the output type the rounding
    # quantum is fixed, so there the two may differ by one quantum).
    out2 = torch.empty_like(out)
    btm.matmul_gpu(a * 2, b, out2)
    tiny = 2.0 ** -14 if dtype == _lib.F16 else 2.0 ** -126
    normal = out.float().abs() > tiny  # strictly: a value that rounded UP to the smallest normal is still a subnormal case
    assert torch.equal(out2[normal], (out * 2)[normal])
    quantum = 2.0 ** -24 if dtype == _lib.F16 else 2.0 ** -133
    assert (out2.float() - out.float() * 2).abs().max().item() <= quantum


def test_repeatable(btm):
    import torch
    a = torch.randn((512, 512), device="cuda").half()
    b = torch.randn((512, 512), device="cuda").half()
    o1, o2 = torch.empty_like(a), torch.empty_like(a)
    btm.matmul_gpu(a, b, o1)
    btm.matmul_gpu(a, b, o2)
    assert torch.equal(o1, o2)


@pytest.mark.parametrize("kernel", ["1cta", "2cta"])
@pytest.mark.parametrize("dtype", [_lib.F16, _lib.BF16])
def test_both_tensor_core_kernels_on_ragged_and_tail_shapes(btm, oracle, dtype, kernel, monkeypatch):
    # The library picks between single CTAs and CTA pairs by size; pin each in turn. The shapes
    # include ones whose last wave is split into half-width tiles (e.g. 38 or 75 full tiles).
    monkeypatch.setenv("BTM_FORCE_KERNEL", kernel)
    for (M, N, K) in [(256, 256, 64), (130, 72, 40), (1000, 1000, 992), (2432, 4096, 128), (384, 6400, 192), (257, 513, 136)]:
        err, _, _ = run_case(btm, oracle, dtype, M, N, K, seed=M + N + K)
        assert err <= TOL[dtype], (kernel, (M, N, K), err)


@pytest.mark.parametrize("dtype", [_lib.F16, _lib.BF16])
def test_transposed_b_entry_point(btm, oracle, dtype):
    # btm_gemm_bt: C = A . Bt^T with Bt stored [N,K]; compared with the oracle on B = Bt^T.
    import ctypes as C
    import torch
    L = _lib.lib()
    for (M, N, K) in [(128, 256, 64), (300, 520, 200), (1024, 1024, 1024), (129, 8, 72)]:
        A, B = gemm_inputs(dtype, M, N, K, 5)
        Bt = np.ascontiguousarray(B.T)
        a, bt = to_gpu(A, dtype), to_gpu(Bt, dtype)
        out = torch.full((M, N), float("nan"), dtype=torch_dtype(dtype), device="cuda")
        rc = L.btm_gemm_bt(0, C.c_void_p(torch.cuda.current_stream().cuda_stream), dtype, M, N, K, a.data_ptr(), K, bt.data_ptr(), K,
                           out.data_ptr(), N)
        assert rc == _lib.OK, _lib.last_error()
        btm.check_device_status(0)
        assert oracle.rel_frobenius(to_host_bits(out, dtype), dtype, oracle.gemm(dtype, A, B)) <= TOL[dtype], (M, N, K)
    # unaligned pitch is refused, not silently mishandled
    a = torch.zeros((8, 12), dtype=torch_dtype(dtype), device="cuda")
    rc = L.btm_gemm_bt(0, None, dtype, 8, 8, 12, a.data_ptr(), 12, a.data_ptr(), 12, a.data_ptr(), 8)
    assert rc == _lib.ERR_UNSUPPORTED


def test_concurrent_callers_on_their_own_streams(btm, oracle):
    # The reference serves operators from pool threads (Helper/Threads/CPUThreading.h:37-56): calls for
    # different tensors may arrive concurrently. Four host threads, each with its own stream and operands.
    import threading
    import torch
    dtype = _lib.F16
    shapes = [(384, 512, 256), (1000, 1000, 992), (257, 513, 136), (512, 2048, 512)]
    results, errors = {}, []

    def worker(i):
        try:
            M, N, K = shapes[i]
            A, B = gemm_inputs(dtype, M, N, K, 50 + i)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                a, b = to_gpu(A, dtype), to_gpu(B, dtype)
                out = torch.empty((M, N), dtype=torch.float16, device="cuda")
                for _ in range(10):
                    btm.matmul_gpu(a, b, out)
                stream.synchronize()
            results[i] = (to_host_bits(out, dtype), A, B)
        except Exception as e:  # surfaced below, in the main thread
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    btm.check_device_status(0)
    for i in range(4):
        got, A, B = results[i]
        assert oracle.rel_frobenius(got, dtype, oracle.gemm(dtype, A, B)) <= TOL[dtype], shapes[i]


def test_concurrent_fp32_callers_with_growing_shapes(btm, oracle):
    # fp32 products need scratch. Each call gets its own block in stream order, so four host threads on four
    # streams with different shapes (a small one first, larger ones after it, so that later calls need more
    # scratch than earlier ones were given) must not disturb one another.
    import threading
    import torch
    dtype = _lib.F32
    shapes = [[(64, 64, 64), (512, 384, 256), (1024, 1024, 512)], [(128, 256, 128), (1000, 1000, 992), (256, 256, 256)],
              [(96, 160, 40), (768, 512, 1024), (1536, 512, 256)], [(257, 129, 65), (384, 2048, 512), (640, 640, 640)]]
    results, errors = {}, []

    def worker(i):
        try:
            stream = torch.cuda.Stream()
            got = []
            with torch.cuda.stream(stream):
                for rep in range(3):
                    for (M, N, K) in shapes[i]:
                        A, B = gemm_inputs(dtype, M, N, K, 90 + i, "uniform")
                        a, b = to_gpu(A, dtype), to_gpu(B, dtype)
                        out = torch.empty((M, N), dtype=torch.float32, device="cuda")
                        btm.matmul_gpu(a, b, out)
                        if rep == 2:
                            got.append((out, A, B))
                stream.synchronize()
            results[i] = [(to_host_bits(o, dtype), A, B) for (o, A, B) in got]
        except Exception as e:  # surfaced below, in the main thread
            errors.append(e)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    btm.check_device_status(0)
    for i in range(4):
        for (got, A, B), shape in zip(results[i], shapes[i]):
            assert oracle.rel_frobenius(got, dtype, oracle.gemm(dtype, A, B)) <= TOL[dtype], shape


def test_fp32_non_finite_inputs(btm):
    # One infinite element makes its output row / column infinite, not NaN (the low half of the split of an
    # infinity is 0, not Inf - Inf); a NaN input still poisons what it touches and nothing else.
    import torch
    M = N = K = 128
    a = torch.rand((M, K), dtype=torch.float32, device="cuda") + 0.5
    b = torch.rand((K, N), dtype=torch.float32, device="cuda") + 0.5
    a[3, 5] = float("inf")
    b[7, 9] = float("-inf")
    a[100, 1] = float("nan")
    out = torch.empty((M, N), dtype=torch.float32, device="cuda")
    btm.matmul_gpu(a, b, out)
    btm.check_device_status(0)
    ref = a.double() @ b.double()
    assert torch.equal(torch.isnan(out), torch.isnan(ref))
    assert torch.equal(torch.isposinf(out), torch.isposinf(ref))
    assert torch.equal(torch.isneginf(out), torch.isneginf(ref))
    fin = torch.isfinite(ref)
    assert ((out.double() - ref)[fin].norm() / ref[fin].norm()).item() <= 1e-5


def test_fp32_with_caller_owned_scratch(btm, oracle):
    import ctypes as C
    import torch
    L = _lib.lib()
    M, N, K = 300, 200, 130
    A, B = gemm_inputs(_lib.F32, M, N, K, 5, "uniform")
    a, b = to_gpu(A, _lib.F32), to_gpu(B, _lib.F32)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    need = L.btm_gemm_f32_workspace_bytes(M, N, K)
    assert need == (M + N) * 132 * 8
    ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    base = (ws.data_ptr() + 255) & ~255
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.btm_gemm_f32_ws(0, st, M, N, K, a.data_ptr(), K, b.data_ptr(), N, out.data_ptr(), N, base, need) == _lib.OK, _lib.last_error()
    btm.check_device_status(0)
    assert oracle.rel_frobenius(to_host_bits(out, _lib.F32), _lib.F32, oracle.gemm(_lib.F32, A, B)) <= 1e-5
    # too small or misaligned scratch is refused
    assert L.btm_gemm_f32_ws(0, st, M, N, K, a.data_ptr(), K, b.data_ptr(), N, out.data_ptr(), N, base, need - 1) == _lib.ERR_INVALID
    assert L.btm_gemm_f32_ws(0, st, M, N, K, a.data_ptr(), K, b.data_ptr(), N, out.data_ptr(), N, base + 8, need) == _lib.ERR_INVALID


@pytest.mark.parametrize("dtype", [_lib.F16, _lib.F32])
def test_user_level_matmul_and_views_with_an_offset(btm, oracle, dtype):
    # ops.matmul allocates the result and dispatches by rank (the Ops::add sketch's style); operands that are
    # views into a larger allocation (offset != 0, row pitch larger than the row) go through unchanged.
    import torch
    M, N, K = 200, 264, 136
    A, B = gemm_inputs(dtype, M, N, K, 41, "uniform" if dtype == _lib.F32 else "normal")
    big_a = torch.zeros((M + 3, K + 24), dtype=torch_dtype(dtype), device="cuda")
    big_b = torch.zeros((K + 2, N + 8), dtype=torch_dtype(dtype), device="cuda")
    big_a[3:, 16:16 + K] = to_gpu(A, dtype)
    big_b[2:, 8:8 + N] = to_gpu(B, dtype)
    a, b = big_a[3:, 16:16 + K], big_b[2:, 8:8 + N]
    assert a.storage_offset() != 0 and b.storage_offset() != 0
    out = btm.matmul(a, b)
    btm.check_device_status(0)
    assert out.shape == (M, N) and out.dtype == torch_dtype(dtype)
    ref = oracle.gemm(dtype, A, B)
    assert oracle.rel_frobenius(to_host_bits(out, dtype), dtype, ref) <= TOL[dtype]
    if dtype == _lib.F16:
        A3 = np.stack([A, A[::-1].copy()])
        B3 = np.stack([B, B[:, ::-1].copy()])
        out3 = btm.matmul(to_gpu(A3, dtype), to_gpu(B3, dtype))
        assert out3.shape == (2, M, N)
        assert oracle.rel_frobenius(to_host_bits(out3, dtype), dtype, oracle.bmm(dtype, A3, B3)) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [_lib.F16, _lib.BF16, _lib.F32])
@pytest.mark.parametrize("layout", ["at", "bt", "at_bt", "strided", "at_unaligned"])
def test_transposed_and_strided_operands_without_a_copy(btm, oracle, dtype, layout):
    # matmul(transpose(a), b), matmul(a, transpose(b)), both, and views with arbitrary strides: Tensor::strides are
    # honoured (Tensor/Tensor.h:173-195) instead of asking the caller to materialise the operand.
    import torch
    shapes = [(256, 384, 192), (300, 200, 130), (128, 136, 72)] if layout != "at_unaligned" else [(131, 77, 53)]
    for (M, N, K) in shapes:
        A, B = gemm_inputs(dtype, M, N, K, 61 + M, "uniform" if dtype == _lib.F32 else "normal")
        a, b = to_gpu(A, dtype), to_gpu(B, dtype)
        if layout in ("at", "at_bt", "at_unaligned"):
            a = a.t().contiguous().t()          # stored [K, M]: unit stride along m
            assert a.stride(0) == 1
        if layout in ("bt", "at_bt"):
            b = b.t().contiguous().t()          # stored [N, K]: unit stride along k
            assert b.stride(1) == K and b.stride(0) == 1
        if layout == "strided":
            big_a = torch.zeros((2 * M, 3 * K), dtype=torch_dtype(dtype), device="cuda")
            big_b = torch.zeros((2 * K, 2 * N), dtype=torch_dtype(dtype), device="cuda")
            big_a[::2, ::3] = a
            big_b[::2, ::2] = b
            a, b = big_a[::2, ::3], big_b[::2, ::2]
        out = torch.full((M, N), float("nan"), dtype=torch_dtype(dtype), device="cuda")
        btm.matmul_gpu(a, b, out)
        btm.check_device_status(0)
        err = oracle.rel_frobenius(to_host_bits(out, dtype), dtype, oracle.gemm(dtype, A, B))
        assert err <= TOL[dtype], (layout, (M, N, K), err)


@pytest.mark.parametrize("kind", ["1cta", "2cta", "fp32"])
def test_chained_products_order(btm, kind, monkeypatch):
    # The products are launched with programmatic stream serialisation: a product may become resident and set itself up
    # while its predecessor still runs, but it reads its operands and writes its output only after the predecessor has
    # completed. A chain C1 = A.B1, C2 = C1.B2, A' = C2 (the next round's output lands in a buffer the chain reads),
    # launched back to back many times, must give bit for bit what it gives with a synchronisation after every launch.
    import torch
    if kind != "fp32":
        monkeypatch.setenv("BTM_FORCE_KERNEL", kind)
    dt = torch.float32 if kind == "fp32" else torch.float16
    n = 768
    g = torch.Generator(device="cuda").manual_seed(11)
    a = (torch.rand((n, n), device="cuda", generator=g) - 0.5).to(dt)
    b1 = (torch.rand((n, n), device="cuda", generator=g) * (2.0 / n ** 0.5)).to(dt)
    b2 = (torch.rand((n, n), device="cuda", generator=g) * (2.0 / n ** 0.5)).to(dt)
    c1, c2, c3 = (torch.zeros((n, n), device="cuda", dtype=dt) for _ in range(3))

    def chain(sync):
        for buf in (c1, c2, c3):
            buf.zero_()
        for _ in range(3):
            btm.matmul_gpu(a, b1, c1)
            if sync:
                torch.cuda.synchronize()
            btm.matmul_gpu(c1, b2, c2)
            if sync:
                torch.cuda.synchronize()
            btm.matmul_gpu(c2, b1, c3)  # reads what the previous launch wrote ...
            if sync:
                torch.cuda.synchronize()
            btm.matmul_gpu(c3, b2, c1)  # ... and overwrites a buffer an earlier launch of the chain read
            if sync:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        return c1.clone(), c2.clone(), c3.clone()

    want = chain(sync=True)
    assert all(torch.isfinite(w).all() for w in want)
    for _ in range(20):
        got = chain(sync=False)
        for w, x in zip(want, got):
            assert torch.equal(w, x)
    btm.check_device_status(0)
