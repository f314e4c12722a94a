"""ctypes front end of the CPU checker (oracle/btm_oracle.c). TEST INFRASTRUCTURE ONLY.

Only the test suite, the smoke check and the CPU-baseline leg of the benchmark import this
module; the shipped package never does. PARITY UNPINNED: the reference project has no
matmul to compare with (Ops/Algebra/MatMul/MatMul.h:1-8 is an empty include guard), so the
arithmetic checked here is the textbook product in binary64; see the header of
btm_oracle.c for what the reference does pin (dtype ordinals, layout, rounding, RNG).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libbtm_oracle.so")

BF16, F16, F32, F64 = 0, 1, 2, 3  # Tensor/Dtypes.h:57-70
_NP = {BF16: np.uint16, F16: np.uint16, F32: np.float32, F64: np.float64}


def build(force: bool = False) -> str:
    """Compile the C restatement (and, if the reference tree is present, oracle/_ref)."""
    src = os.path.join(_HERE, "btm_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libbtm_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


def build_ref(ref_root: str | None = None) -> str | None:
    """Compile the reference's own Tensor::random driver when its sources are present. The reference tree is
    `ref_root`, else the environment variable BTM_REFERENCE_ROOT, else a directory named `reference` beside this
    repository; without any of them only an already built driver is returned."""
    out = os.path.join(_HERE, "_ref", "ref_random")
    if os.path.exists(out):
        return out
    sibling = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    ref_root = ref_root or os.environ.get("BTM_REFERENCE_ROOT") or sibling
    if not os.path.isfile(os.path.join(ref_root, "Tensor", "Tensor.cpp")):
        return None
    subprocess.check_call(["make", "-C", _HERE, "ref", f"REF={ref_root}"], stdout=subprocess.DEVNULL)
    return out


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        i64, vp, dbl = C.c_int64, C.c_void_p, C.c_double
        L.btmo_gemm.argtypes = [C.c_int, i64, i64, i64, vp, i64, vp, i64, vp, i64, C.c_int]
        L.btmo_bmm.argtypes = [C.c_int, i64, i64, i64, i64, vp, i64, vp, i64, vp, i64, C.c_int]
        L.btmo_int4_pack.argtypes = [vp, i64, i64, vp]
        L.btmo_int4_unpack.argtypes = [vp, i64, i64, vp]
        L.btmo_int4_dequant.argtypes = [vp, vp, i64, i64, i64, vp]
        L.btmo_int4_matmul.argtypes = [i64, i64, i64, i64, vp, vp, vp, vp, C.c_int]
        L.btmo_int4_quantize.argtypes = [vp, i64, i64, i64, vp, vp]
        L.btmo_rel_frobenius.argtypes = [vp, C.c_int, vp, C.c_size_t]
        L.btmo_rel_frobenius.restype = dbl
        L.btmo_widen.argtypes = [vp, C.c_int, C.c_size_t, vp]
        L.btmo_narrow.argtypes = [vp, C.c_int, C.c_size_t, vp]
        L.btmo_ref_random_f32.argtypes = [vp, C.c_size_t, C.c_uint64, dbl, dbl, C.c_int]
        L.btmo_ref_random_f64.argtypes = [vp, C.c_size_t, C.c_uint64, dbl, dbl, C.c_int]
        L.btmo_gemm_f32_threads.argtypes = [i64, i64, i64, vp, vp, vp, C.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray) -> C.c_void_p:
    assert a.flags["C_CONTIGUOUS"]
    return C.c_void_p(a.ctypes.data)


def threads() -> int:
    return max(1, min(os.cpu_count() or 1, 64))


def gemm(dtype: int, A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """C = A.B in binary64 from `dtype` storage (uint16 bit patterns for fp16/bf16)."""
    M, K = A.shape
    K2, N = B.shape
    assert K == K2 and A.dtype == _NP[dtype] and B.dtype == _NP[dtype]
    A = np.ascontiguousarray(A)
    B = np.ascontiguousarray(B)
    out = np.zeros((M, N), dtype=np.float64)
    rc = lib().btmo_gemm(dtype, M, N, K, _p(A), K, _p(B), N, _p(out), N, threads())
    assert rc == 0
    return out


def bmm(dtype: int, A: np.ndarray, B: np.ndarray) -> np.ndarray:
    b, M, K = A.shape
    b2, K2, N = B.shape
    assert b == b2 and K == K2
    A = np.ascontiguousarray(A)
    B = np.ascontiguousarray(B)
    out = np.zeros((b, M, N), dtype=np.float64)
    rc = lib().btmo_bmm(dtype, b, M, N, K, _p(A), M * K, _p(B), K * N, _p(out), M * N, threads())
    assert rc == 0
    return out


def int4_pack(w: np.ndarray) -> np.ndarray:
    N, K = w.shape
    w = np.ascontiguousarray(w.astype(np.int8))
    out = np.zeros((N, K // 2), dtype=np.uint8)
    lib().btmo_int4_pack(_p(w), N, K, _p(out))
    return out


def int4_unpack(packed: np.ndarray) -> np.ndarray:
    N, K2 = packed.shape
    out = np.zeros((N, K2 * 2), dtype=np.int8)
    lib().btmo_int4_unpack(_p(np.ascontiguousarray(packed)), N, K2 * 2, _p(out))
    return out


def int4_dequant(packed: np.ndarray, scales_f16: np.ndarray, group: int) -> np.ndarray:
    N, K2 = packed.shape
    K = K2 * 2
    out = np.zeros((N, K), dtype=np.uint16)
    lib().btmo_int4_dequant(_p(np.ascontiguousarray(packed)), _p(np.ascontiguousarray(scales_f16)), N, K, group, _p(out))
    return out


def int4_matmul(act_f16: np.ndarray, packed: np.ndarray, scales_f16: np.ndarray, group: int) -> np.ndarray:
    M, K = act_f16.shape
    N = packed.shape[0]
    out = np.zeros((M, N), dtype=np.float64)
    rc = lib().btmo_int4_matmul(M, N, K, group, _p(np.ascontiguousarray(act_f16)), _p(np.ascontiguousarray(packed)),
                                _p(np.ascontiguousarray(scales_f16)), _p(out), threads())
    assert rc == 0
    return out


def int4_quantize(w_f16: np.ndarray, group: int):
    """fp16 bit patterns [N,K] -> (packed [N,K/2] bytes, scales [N,K/group] fp16 bit patterns)."""
    N, K = w_f16.shape
    packed = np.zeros((N, K // 2), dtype=np.uint8)
    scales = np.zeros((N, K // group), dtype=np.uint16)
    lib().btmo_int4_quantize(_p(np.ascontiguousarray(w_f16)), N, K, group, _p(packed), _p(scales))
    return packed, scales


def rel_frobenius(X: np.ndarray, dtype: int, R: np.ndarray) -> float:
    X = np.ascontiguousarray(X)
    R = np.ascontiguousarray(R, dtype=np.float64)
    assert X.size == R.size
    return float(lib().btmo_rel_frobenius(_p(X), dtype, _p(R), X.size))


def narrow(x64: np.ndarray, dtype: int) -> np.ndarray:
    x64 = np.ascontiguousarray(x64, dtype=np.float64)
    out = np.zeros(x64.shape, dtype=_NP[dtype])
    lib().btmo_narrow(_p(x64), dtype, x64.size, _p(out))
    return out


def widen(x: np.ndarray, dtype: int) -> np.ndarray:
    x = np.ascontiguousarray(x)
    out = np.zeros(x.shape, dtype=np.float64)
    lib().btmo_widen(_p(x), dtype, x.size, _p(out))
    return out


def ref_random_f32(shape, seed: int, lo: float, hi: float, ref_threads: int) -> np.ndarray:
    """Restatement of the reference's Tensor::random for fp32 (Tensor/Tensor.cpp:89-152)."""
    out = np.zeros(shape, dtype=np.float32)
    lib().btmo_ref_random_f32(_p(out), out.size, seed, lo, hi, ref_threads)
    return out


def gemm_f32_threads(A: np.ndarray, B: np.ndarray, nthreads: int) -> np.ndarray:
    """Timed CPU baseline body: fp32 blocked matmul on `nthreads` host threads."""
    M, K = A.shape
    N = B.shape[1]
    out = np.empty((M, N), dtype=np.float32)
    lib().btmo_gemm_f32_threads(M, N, K, _p(A), _p(B), _p(out), nthreads)
    return out
