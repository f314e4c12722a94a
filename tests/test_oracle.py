"""Pins the CPU checker (oracle/) against the committed golden vectors. No GPU."""
import hashlib
import os

import numpy as np

from beantensor_b200 import _lib

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_reference_rng_restatement_matches_reference_output(oracle):
    # Golden vectors were produced by the reference's own Tensor::random (Tensor/Tensor.cpp:268-298).
    g = np.load(os.path.join(GOLD, "ref_random.npz"))
    threads = int(g["threads"][0])
    for name in ("a", "b", "c"):
        rows, cols, seed, lo, hi = g[name + "_args"]
        mine = oracle.ref_random_f32((int(rows), int(cols)), int(seed), float(lo), float(hi), threads)
        assert np.array_equal(mine, g[name]), name
    cfg1 = oracle.ref_random_f32((1024, 1024), 0, -1.0, 1.0, threads)
    assert np.array_equal(cfg1.ravel()[:16], g["cfg1_head"])
    digest = np.frombuffer(hashlib.sha256(cfg1.tobytes()).digest(), dtype=np.uint8)
    assert np.array_equal(digest, g["cfg1_sha256"])


def test_reference_rng_chunking_depends_on_thread_count(oracle):
    # Tensor/Tensor.cpp:141-151: chunk t is seeded seed+t; a single stream below threads*1024 elements.
    one = oracle.ref_random_f32((64, 64), 3, -1.0, 1.0, 8)
    also_one = oracle.ref_random_f32((64, 64), 3, -1.0, 1.0, 4)
    assert np.array_equal(one, also_one)  # 4096 <= 4*1024: single stream either way
    big8 = oracle.ref_random_f32((128, 128), 3, -1.0, 1.0, 8)
    big4 = oracle.ref_random_f32((128, 128), 3, -1.0, 1.0, 4)
    assert not np.array_equal(big8, big4)
    # chunk 1 of the 8-thread fill starts with the first draw of seed+1
    assert big8.ravel()[2048] == oracle.ref_random_f32((1, 1), 4, -1.0, 1.0, 8)[0, 0]


def test_narrowing_is_rne(oracle):
    g = np.load(os.path.join(GOLD, "narrow.npz"))
    assert np.array_equal(oracle.narrow(g["x"], oracle.F16), g["f16"])
    assert np.array_equal(oracle.narrow(g["x"], oracle.BF16), g["bf16"])
    back = oracle.widen(g["f16"], oracle.F16)
    finite = np.isfinite(back)
    assert np.array_equal(back[finite], g["f16"].view(np.float16).astype(np.float64)[finite])


def test_gemm_against_numpy_golden(oracle):
    g = np.load(os.path.join(GOLD, "gemm_small.npz"))
    for i in range(int(g["ncases"][0])):
        dt, M, N, K = (int(v) for v in g[f"case{i}_meta"])
        C = oracle.gemm(dt, g[f"case{i}_A"], g[f"case{i}_B"])
        want = g[f"case{i}_C"]
        assert C.shape == want.shape == (M, N)
        # both accumulate in fp64; only the summation order differs
        assert np.allclose(C, want, rtol=0, atol=1e-13 * max(K, 1)), i


def test_int4_against_numpy_golden(oracle):
    g = np.load(os.path.join(GOLD, "int4_small.npz"))
    for i in range(int(g["ncases"][0])):
        M, N, K, group = (int(v) for v in g[f"case{i}_meta"])
        w, packed = g[f"case{i}_w"], g[f"case{i}_packed"]
        assert np.array_equal(oracle.int4_pack(w), packed)
        assert np.array_equal(oracle.int4_unpack(packed), w)
        assert np.array_equal(oracle.int4_dequant(packed, g[f"case{i}_scales"], group), g[f"case{i}_dequant"])
        out = oracle.int4_matmul(g[f"case{i}_act"], packed, g[f"case{i}_scales"], group)
        assert np.allclose(out, g[f"case{i}_out"], rtol=0, atol=1e-9)


def test_bmm_is_per_batch_gemm(oracle):
    from tests.helpers import gemm_inputs
    A, B = gemm_inputs(_lib.F16, 3 * 16, 24, 32, 5)
    A3 = A.reshape(3, 16, 32)
    B3 = np.stack([B, B[::-1].copy(), B * 0 + B[0:1]])
    C = oracle.bmm(_lib.F16, A3, B3)
    for b in range(3):
        assert np.array_equal(C[b], oracle.gemm(_lib.F16, A3[b], B3[b]))


def test_rel_frobenius(oracle):
    R = np.array([[3.0, 4.0]])
    X = np.array([[3.0, 4.0]], dtype=np.float32)
    assert oracle.rel_frobenius(X, oracle.F32, R) == 0.0
    X2 = np.array([[3.0, 4.5]], dtype=np.float32)
    assert abs(oracle.rel_frobenius(X2, oracle.F32, R) - 0.1) < 1e-12


def test_cpu_baseline_body_matches_oracle(oracle):
    from beantensor_b200 import synth
    A = synth.uniform((96, 80), -1, 1, 1, 0).astype(np.float32)
    B = synth.uniform((80, 72), -1, 1, 1, 1).astype(np.float32)
    C = oracle.gemm_f32_threads(A, B, 3)
    assert oracle.rel_frobenius(C, oracle.F32, oracle.gemm(oracle.F32, A, B)) < 1e-6


def test_quantiser_restatement_against_numpy(oracle):
    from beantensor_b200 import synth
    N, K, group = 12, 256, 64
    w = synth.normal((N, K), 0.05, 77, 0).astype(np.float16)
    w[3, :group] = 0
    packed, scales = oracle.int4_quantize(w.view(np.uint16), group)
    wf = w.astype(np.float32).reshape(N, K // group, group)
    s = (np.abs(wf).max(axis=2) / np.float32(7.0)).astype(np.float16)
    s[s == 0] = np.float16(1.0)
    assert np.array_equal(scales, s.view(np.uint16))
    q = np.clip(np.rint(wf / s.astype(np.float32)[:, :, None]), -8, 7).astype(np.int8).reshape(N, K)
    assert np.array_equal(oracle.int4_unpack(packed), q)
