"""Shared helpers of the parity tests: seeded inputs in storage format and GPU plumbing."""
from __future__ import annotations

import numpy as np

from beantensor_b200 import _lib, synth

NP_STORE = {_lib.F16: np.uint16, _lib.BF16: np.uint16, _lib.F32: np.float32}
# Tolerances of the path (relative Frobenius error against the fp64 oracle).
TOL = {_lib.F16: 2e-3, _lib.BF16: 2e-3, _lib.F32: 1e-5}


def store(x64: np.ndarray, dtype: int) -> np.ndarray:
    """fp64 values -> storage bit patterns of `dtype` (RNE)."""
    if dtype == _lib.F32:
        return x64.astype(np.float32)
    if dtype == _lib.F16:
        return synth.to_f16_bits(x64.astype(np.float32))
    return synth.to_bf16_bits(x64.astype(np.float32))


def torch_dtype(dtype: int):
    import torch
    return {_lib.F16: torch.float16, _lib.BF16: torch.bfloat16, _lib.F32: torch.float32}[dtype]


def to_gpu(bits: np.ndarray, dtype: int):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(bits))
    if dtype in (_lib.F16, _lib.BF16):
        t = t.view(torch_dtype(dtype))
    return t.cuda()


def to_host_bits(t, dtype: int) -> np.ndarray:
    import torch
    t = t.detach().cpu().contiguous()
    if dtype in (_lib.F16, _lib.BF16):
        return t.view(torch.uint16).numpy()
    return t.numpy()


def gemm_inputs(dtype: int, M: int, N: int, K: int, seed: int, dist: str = "normal"):
    if dist == "uniform":
        A = synth.uniform((M, K), -1.0, 1.0, seed, 0)
        B = synth.uniform((K, N), -1.0, 1.0, seed, 1)
    else:
        std = 1.0 / np.sqrt(max(K, 1))
        A = synth.normal((M, K), std, seed, 0)
        B = synth.normal((K, N), std, seed, 1)
    return store(A, dtype), store(B, dtype)
