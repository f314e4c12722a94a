"""Regenerates the committed golden vectors (run from the repository root, in a container that
has the reference tree): python tests/golden/make_golden.py

What is pinned, and against what:
  ref_random.npz   outputs of the REFERENCE'S OWN Tensor::random (Tensor/Tensor.cpp:268-298),
                   produced by oracle/_ref/ref_random, a driver compiled from the reference
                   sources where they lie. Pins the oracle's restatement of that generator.
  narrow.npz       fp64 -> fp16/bf16 round-to-nearest-even bit patterns from numpy / torch.
                   Pins the rounding the reference's CUDA path uses (Tensor/TensorOps.cu:72).
  gemm_small.npz   small products in every supported dtype; expected results by numpy float64
                   matmul, which is independent of the oracle's C code.
  int4_small.npz   packed weights, scales, activations; expected unpack / dequant / product by
                   numpy.
The reference has no matmul, so nothing else of this path can be pinned to it.
"""
import hashlib
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
OUT = os.path.dirname(os.path.abspath(__file__))

from beantensor_b200 import _lib, synth  # noqa: E402
from oracle import oracle as O  # noqa: E402
from tests.helpers import store  # noqa: E402


def ref_random():
    exe = O.build_ref()
    assert exe, "reference tree not present"
    out = {}
    threads = None
    for name, rows, cols, seed, lo, hi in [("a", 4, 5, 7, -1.0, 1.0), ("b", 96, 97, 0, -1.0, 1.0), ("c", 33, 1000, 42, 500.0, 600.0)]:
        r = subprocess.run([exe, str(rows), str(cols), str(seed), str(lo), str(hi)], capture_output=True, check=True)
        threads = int(r.stderr.decode().split("threads=")[1].split()[0])
        out[name] = np.frombuffer(r.stdout, dtype=np.float32).reshape(rows, cols).copy()
        out[name + "_args"] = np.array([rows, cols, seed, lo, hi], dtype=np.float64)
    # The 1024 x 1024, seed 0, U[-1,1] matrix of the reference's CPU-runnable workload: digest only.
    r = subprocess.run([exe, "1024", "1024", "0", "-1", "1"], capture_output=True, check=True)
    out["cfg1_sha256"] = np.frombuffer(hashlib.sha256(r.stdout).digest(), dtype=np.uint8)
    out["cfg1_head"] = np.frombuffer(r.stdout, dtype=np.float32)[:16].copy()
    out["threads"] = np.array([threads])
    np.savez_compressed(os.path.join(OUT, "ref_random.npz"), **out)


def narrow():
    import torch
    rng = np.random.default_rng(123)
    x = rng.standard_normal(4096) * np.exp(rng.uniform(-30, 12, 4096))
    x32 = x.astype(np.float32).astype(np.float64)  # fp32-representable, so torch's path rounds once
    special = np.array([0.0, -0.0, 65504.0, 65520.0, 65519.99, 6e-8, 2.98e-8, 2.9802322387695312e-08, 1.0009765625,
                        1.00048828125, 1.00146484375, -1.00048828125, 3.3e38, 1e-45])
    x32 = np.concatenate([x32, special.astype(np.float32).astype(np.float64)])
    f16 = x32.astype(np.float16).view(np.uint16)
    bf16 = torch.from_numpy(x32.astype(np.float32)).to(torch.bfloat16).view(torch.uint16).numpy()
    np.savez_compressed(os.path.join(OUT, "narrow.npz"), x=x32, f16=f16, bf16=bf16)


def widen_np(bits, dtype):
    if dtype == _lib.F32:
        return bits.astype(np.float64)
    if dtype == _lib.F16:
        return bits.view(np.float16).astype(np.float64)
    return (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def gemm_small():
    out = {}
    cases = [(_lib.F16, 8, 16, 32), (_lib.F16, 33, 17, 65), (_lib.BF16, 64, 40, 72), (_lib.F32, 31, 29, 57),
             (_lib.F32, 64, 64, 64), (_lib.F16, 1, 1, 1), (_lib.BF16, 5, 3, 0)]
    for i, (dt, M, N, K) in enumerate(cases):
        A = store(synth.normal((M, K), 1.0 / np.sqrt(max(K, 1)), 100 + i, 0), dt)
        B = store(synth.normal((K, N), 1.0 / np.sqrt(max(K, 1)), 100 + i, 1), dt)
        C = widen_np(A, dt) @ widen_np(B, dt)
        out[f"case{i}_meta"] = np.array([dt, M, N, K])
        out[f"case{i}_A"], out[f"case{i}_B"], out[f"case{i}_C"] = A, B, C
    out["ncases"] = np.array([len(cases)])
    np.savez_compressed(os.path.join(OUT, "gemm_small.npz"), **out)


def int4_small():
    out = {}
    cases = [(1, 16, 128, 128), (3, 40, 256, 128), (8, 24, 512, 256), (2, 7, 64, 32)]
    for i, (M, N, K, group) in enumerate(cases):
        w = synth.int4((N, K), 200 + i)
        packed = synth.pack_int4(w)
        s = synth.uniform((N, K // group), 0.005, 0.02, 200 + i, 1).astype(np.float16)
        act = synth.normal((M, K), 1.0, 200 + i, 2).astype(np.float16)
        s_full = np.repeat(s.astype(np.float32), group, axis=1)
        deq = (w.astype(np.float32) * s_full).astype(np.float16)  # exact product, one rounding
        prod = act.astype(np.float64) @ (w.astype(np.float64) * s_full.astype(np.float64)).T
        out[f"case{i}_meta"] = np.array([M, N, K, group])
        out[f"case{i}_w"], out[f"case{i}_packed"] = w, packed
        out[f"case{i}_scales"], out[f"case{i}_act"] = s.view(np.uint16), act.view(np.uint16)
        out[f"case{i}_dequant"], out[f"case{i}_out"] = deq.view(np.uint16), prod
    out["ncases"] = np.array([len(cases)])
    np.savez_compressed(os.path.join(OUT, "int4_small.npz"), **out)


if __name__ == "__main__":
    ref_random()
    narrow()
    gemm_small()
    int4_small()
    for f in sorted(os.listdir(OUT)):
        print(f, os.path.getsize(os.path.join(OUT, f)))
