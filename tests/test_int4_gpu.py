"""int4 weight-only path: bit-exact unpack and dequant, matmul within 2e-3 of the oracle."""
import os

import numpy as np
import pytest

from beantensor_b200 import synth

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def make(M, N, K, group, seed):
    w = synth.int4((N, K), seed)
    packed = synth.pack_int4(w)
    s = synth.uniform((N, K // group), 0.005, 0.02, seed, 1).astype(np.float16)
    act = synth.normal((M, K), 1.0, seed, 2).astype(np.float16)
    return w, packed, s, act


def gpu_matmul(btm, act, packed, s, group):
    import torch
    out = torch.full((act.shape[0], packed.shape[0]), float("nan"), dtype=torch.float16, device="cuda")
    btm.matmul_int4_gpu(torch.from_numpy(act).cuda(), torch.from_numpy(packed).cuda(), torch.from_numpy(s).cuda(), out, group)
    return out.cpu().numpy()


def test_golden_cases_bit_exact_dequant(btm, oracle):
    import torch
    g = np.load(os.path.join(GOLD, "int4_small.npz"))
    for i in range(int(g["ncases"][0])):
        M, N, K, group = (int(v) for v in g[f"case{i}_meta"])
        packed = torch.from_numpy(g[f"case{i}_packed"]).cuda()
        scales = torch.from_numpy(g[f"case{i}_scales"]).view(torch.float16).cuda()
        deq = torch.empty((N, K), dtype=torch.float16, device="cuda")
        btm.dequant_int4_gpu(packed, scales, deq, group)
        assert np.array_equal(deq.cpu().view(torch.uint16).numpy(), g[f"case{i}_dequant"]), i
        unp = torch.empty((N, K), dtype=torch.int8, device="cuda")
        btm.unpack_int4_gpu(packed, unp)
        assert np.array_equal(unp.cpu().numpy(), g[f"case{i}_w"]), i
        act = g[f"case{i}_act"].view(np.float16)
        out = gpu_matmul(btm, act, g[f"case{i}_packed"], g[f"case{i}_scales"].view(np.float16), group)
        assert oracle.rel_frobenius(out.view(np.uint16), oracle.F16, g[f"case{i}_out"]) <= 2e-3, i


@pytest.mark.parametrize("M", [1, 8, 64])
def test_workload_shape(btm, oracle, M):
    # N=11008, K=4096, group 128: the whole weight matrix, bit-exact dequant and 2e-3 output.
    import torch
    N, K, group = 11008, 4096, 128
    w, packed, s, act = make(M, N, K, group, 2)
    out = gpu_matmul(btm, act, packed, s, group)
    ref = oracle.int4_matmul(act.view(np.uint16), packed, s.view(np.uint16), group)
    assert oracle.rel_frobenius(out.view(np.uint16), oracle.F16, ref) <= 2e-3
    if M == 1:
        deq = torch.empty((N, K), dtype=torch.float16, device="cuda")
        btm.dequant_int4_gpu(torch.from_numpy(packed).cuda(), torch.from_numpy(s).cuda(), deq, group)
        assert np.array_equal(deq.cpu().view(torch.uint16).numpy(), oracle.int4_dequant(packed, s.view(np.uint16), group))
        unp = torch.empty((N, K), dtype=torch.int8, device="cuda")
        btm.unpack_int4_gpu(torch.from_numpy(packed).cuda(), unp)
        assert np.array_equal(unp.cpu().numpy(), w)


@pytest.mark.parametrize("case", [(1, 16, 128, 128), (2, 17, 256, 128), (5, 100, 1024, 256), (9, 33, 384, 128),
                                  (3, 40, 96, 32), (1, 5, 64, 64), (8, 16, 8192, 128)])
def test_ragged_and_general_shapes(btm, oracle, case):
    # N not a multiple of 16, M crossing the 8-row block, groups other than 128 (general kernel).
    M, N, K, group = case
    w, packed, s, act = make(M, N, K, group, 17 + M + N)
    out = gpu_matmul(btm, act, packed, s, group)
    assert not np.isnan(out).any()
    ref = oracle.int4_matmul(act.view(np.uint16), packed, s.view(np.uint16), group)
    assert oracle.rel_frobenius(out.view(np.uint16), oracle.F16, ref) <= 2e-3


def test_extreme_nibbles(btm, oracle):
    # all -8, all 7, alternating: exercises the sign handling of the unpack
    import torch
    N, K, group = 32, 256, 128
    for fill in (-8, 7, None):
        w = np.full((N, K), fill if fill is not None else 0, dtype=np.int8)
        if fill is None:
            w[:, 0::2], w[:, 1::2] = -8, 7
        packed = synth.pack_int4(w)
        s = np.full((N, K // group), 0.0078125, dtype=np.float16)
        act = np.ones((2, K), dtype=np.float16)
        out = gpu_matmul(btm, act, packed, s, group)
        want = w.astype(np.float64).sum(axis=1) * 0.0078125
        assert np.allclose(out.astype(np.float64), np.broadcast_to(want, (2, N)), rtol=2e-3)


def test_bad_arguments(btm):
    import torch
    act = torch.zeros((1, 100), dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        btm.matmul_int4_gpu(act, torch.zeros((16, 50), dtype=torch.uint8, device="cuda"),
                            torch.zeros((16, 0), dtype=torch.float16, device="cuda"),
                            torch.zeros((1, 16), dtype=torch.float16, device="cuda"), 128)


@pytest.mark.parametrize("path", ["regs", "stream", "slab"])
@pytest.mark.parametrize("case", [(1, 11008, 4096, 128), (8, 11008, 4096, 128), (3, 100, 4096, 128), (2, 37, 2048, 128),
                                  (1, 48, 2304, 128), (5, 16, 8192, 256), (2, 3000, 4096, 128), (4, 5000, 1024, 128), (7, 129, 11008, 128),
                                  (8, 40, 12288, 512), (6, 2049, 640, 128), (4, 11008, 4096, 128), (1, 700, 512, 128), (3, 31, 3584, 128)])
def test_gemv_both_kernels(btm, oracle, case, path, monkeypatch):
    # M <= 8 pinned to each of the three kernels: register-resident (the default up to four rows), persistent streaming
    # (the default above), one whole 16-row slab per CTA. A kernel that does not take a shape hands it on.
    M, N, K, group = case
    monkeypatch.setenv("BTM_FORCE_GEMV", path)
    w, packed, s, act = make(M, N, K, group, 23 + M + N)
    out = gpu_matmul(btm, act, packed, s, group)
    assert not np.isnan(out).any()
    btm.check_device_status(0)
    ref = oracle.int4_matmul(act.view(np.uint16), packed, s.view(np.uint16), group)
    assert oracle.rel_frobenius(out.view(np.uint16), oracle.F16, ref) <= 2e-3


@pytest.mark.parametrize("path", ["tensor_core", "mma"])
@pytest.mark.parametrize("case", [(16, 128, 256, 128), (64, 1088, 1024, 128), (100, 200, 512, 64), (129, 72, 1024, 256), (40, 64, 4096, 128),
                                  (16, 19200, 256, 128), (24, 12800, 512, 128), (20, 33, 384, 128)])
def test_more_than_eight_rows_both_paths(btm, oracle, case, path, monkeypatch):
    # M > 8 runs on tcgen05 (weights dequantised into tensor memory) unless pinned to the mma.sync kernel.
    M, N, K, group = case
    if path == "mma":
        monkeypatch.setenv("BTM_FORCE_INT4", "mma")
    w, packed, s, act = make(M, N, K, group, 31 + M)
    out = gpu_matmul(btm, act, packed, s, group)
    btm.check_device_status(0)
    assert not np.isnan(out).any()
    ref = oracle.int4_matmul(act.view(np.uint16), packed, s.view(np.uint16), group)
    assert oracle.rel_frobenius(out.view(np.uint16), oracle.F16, ref) <= 2e-3
    if path == "tensor_core":
        # The tensor-core path multiplies by the dequantised fp16 weights (the btm_int4_dequant values):
        # against a product of exactly those values only accumulation order and the output rounding differ.
        dq = oracle.int4_dequant(packed, s.view(np.uint16), group)
        ref_dq = oracle.gemm(oracle.F16, act.view(np.uint16), np.ascontiguousarray(dq.T))
        assert oracle.rel_frobenius(out.view(np.uint16), oracle.F16, ref_dq) <= 5e-4


def _seeded_shapes():
    # A fixed pseudo-random walk over shapes that reach every int4 kernel: GEMV (streaming and slab), the
    # tcgen05 kernel with 1..3-way K splits, one and two 128-row passes, partial tiles, several group sizes.
    rng = np.random.default_rng(20240607)
    cases = []
    for _ in range(28):
        M = int(rng.choice([1, 2, 3, 5, 8, 9, 16, 31, 64, 65, 100, 128, 130, 200]))
        K = int(rng.choice([128, 256, 512, 1024, 1536, 2048, 4096]))
        divisors = [g for g in (64, 128, 256, 512, 1024) if K % g == 0]
        group = int(rng.choice(divisors))
        N = int(rng.choice([1, 7, 16, 33, 100, 128, 129, 255, 300, 1000, 2049, 5000]))
        cases.append((M, N, K, group))
    return cases


@pytest.mark.parametrize("case", _seeded_shapes())
def test_seeded_shape_walk(btm, oracle, case):
    M, N, K, group = case
    w, packed, s, act = make(M, N, K, group, 101 + M + N + K)
    out = gpu_matmul(btm, act, packed, s, group)
    assert not np.isnan(out).any()
    btm.check_device_status(0)
    ref = oracle.int4_matmul(act.view(np.uint16), packed, s.view(np.uint16), group)
    assert oracle.rel_frobenius(out.view(np.uint16), oracle.F16, ref) <= 2e-3


@pytest.mark.parametrize("M", [4, 32, 64])
def test_chained_products_order(btm, oracle, M):
    # The int4 products start early under their predecessor (programmatic dependent launch) and may prefetch weights
    # and scales, but activations are read and outputs written only after the predecessor has completed. A chain
    # whose second product consumes the first one's output, launched back to back many times, must give bit for bit
    # what the same chain gives with a synchronisation after every launch.
    import torch
    N1, K1, group = 1024, 1024, 128
    N2 = 768
    _, p1, s1, act = make(M, N1, K1, group, 501 + M)
    _, p2, s2, _ = make(M, N2, N1, group, 502 + M)
    a = torch.from_numpy(act).cuda()
    w1, sc1 = torch.from_numpy(p1).cuda(), torch.from_numpy(s1).cuda()
    w2, sc2 = torch.from_numpy(p2).cuda(), torch.from_numpy(s2).cuda()
    mid = torch.zeros((M, N1), dtype=torch.float16, device="cuda")
    out = torch.zeros((M, N2), dtype=torch.float16, device="cuda")
    btm.matmul_int4_gpu(a, w1, sc1, mid, group)
    torch.cuda.synchronize()
    btm.matmul_int4_gpu(mid, w2, sc2, out, group)
    torch.cuda.synchronize()
    want_mid, want_out = mid.clone(), out.clone()
    ref = oracle.int4_matmul(want_mid.cpu().numpy().view(np.uint16), p2, s2.view(np.uint16), group)
    assert oracle.rel_frobenius(want_out.cpu().numpy().view(np.uint16), oracle.F16, ref) <= 2e-3
    for _ in range(30):
        mid.zero_()
        out.zero_()
        for _ in range(4):
            btm.matmul_int4_gpu(a, w1, sc1, mid, group)
            btm.matmul_int4_gpu(mid, w2, sc2, out, group)
        torch.cuda.synchronize()
        assert torch.equal(mid, want_mid)
        assert torch.equal(out, want_out)
    btm.check_device_status(0)


@pytest.mark.parametrize("case", [(600, 1088, 1024, 128, None), (1024, 264, 512, 64, None), (40, 64, 4096, 128, "16"), (130, 200, 256, 128, "100"),
                                  (600, 1088, 1024, 128, "100000")])
def test_many_rows_take_the_dequantise_once_route(btm, oracle, case, monkeypatch):
    # From 512 activation rows on the weights are dequantised once into scratch and multiplied by the dense tensor-core
    # kernel; below, the tcgen05 int4 kernel unpacks them per 128 rows. Both multiply by the btm_int4_dequant values, so
    # both must agree with a product of exactly those values; the threshold is moved to run small shapes through the
    # scratch route and a large one through the per-pass kernel.
    M, N, K, group, threshold = case
    if threshold:
        monkeypatch.setenv("BTM_INT4_LARGE_M", threshold)
    w, packed, s, act = make(M, N, K, group, 77 + M)
    out = gpu_matmul(btm, act, packed, s, group)
    btm.check_device_status(0)
    assert not np.isnan(out).any()
    ref = oracle.int4_matmul(act.view(np.uint16), packed, s.view(np.uint16), group)
    assert oracle.rel_frobenius(out.view(np.uint16), oracle.F16, ref) <= 2e-3
    dq = oracle.int4_dequant(packed, s.view(np.uint16), group)
    ref_dq = oracle.gemm(oracle.F16, act.view(np.uint16), np.ascontiguousarray(dq.T))
    assert oracle.rel_frobenius(out.view(np.uint16), oracle.F16, ref_dq) <= 5e-4
