"""Seeded synthetic inputs for the matmul workloads.

The reference's generator (Tensor::random, Tensor/Tensor.cpp:89-152) is uniform-only and its
stream depends on the host's thread count, so the workloads that ask for normal or int4 inputs
use this counter-based generator instead: every value is a pure function of (seed, stream,
flat index), independent of how the work is split. splitmix64 finaliser as the mixer.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = (z + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def bits(seed: int, stream: int, n: int, lane: int = 0) -> np.ndarray:
    """n 64-bit draws: draw i = mix(key + i*golden) with key = mix(mix(seed) ^ stream*odd + lane)."""
    key = _mix(np.array([seed], dtype=np.uint64))
    with np.errstate(over="ignore"):
        key = _mix(key ^ (np.uint64(stream) * np.uint64(0xD1B54A32D192ED03) + np.uint64(lane)))
        idx = np.arange(n, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)
        return _mix(key + idx)


def uniform01(seed: int, stream: int, n: int, lane: int = 0) -> np.ndarray:
    return (bits(seed, stream, n, lane) >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def uniform(shape, lo: float, hi: float, seed: int, stream: int = 0) -> np.ndarray:
    n = int(np.prod(shape))
    return (uniform01(seed, stream, n) * (hi - lo) + lo).reshape(shape)


def normal(shape, std: float, seed: int, stream: int = 0) -> np.ndarray:
    """Box-Muller on two independent draws per element; mean 0, standard deviation `std`."""
    n = int(np.prod(shape))
    u1 = 1.0 - uniform01(seed, stream, n, lane=0)  # (0, 1]
    u2 = uniform01(seed, stream, n, lane=1)
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2) * std).reshape(shape)


def int4(shape, seed: int, stream: int = 0) -> np.ndarray:
    """Signed 4-bit values uniform in [-8, 7] as int8."""
    n = int(np.prod(shape))
    return ((bits(seed, stream, n) >> np.uint64(60)).astype(np.int16) - 8).astype(np.int8).reshape(shape)


def pack_int4(w: np.ndarray) -> np.ndarray:
    """[N,K] int8 in [-8,7] -> [N,K/2] bytes, even k in bits 0-3, odd k in bits 4-7."""
    u = (w.astype(np.int16) & 0xF).astype(np.uint8)
    return (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bfloat16 bit patterns, round to nearest even (finite inputs)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def to_f16_bits(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x).astype(np.float16).view(np.uint16)
