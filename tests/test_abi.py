"""CPU-side checks of the boundary: the library loads and exports exactly what include/btm.h
declares; argument validation answers before any CUDA work. No compute call needs a GPU here."""
import ctypes
import os
import re

from beantensor_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "btm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(btm_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    L = _lib.lib()
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/btm.h but not exported by libbtm.so"


def test_binding_covers_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_dtype_sizes_follow_reference_enum():
    # Tensor/Dtypes.h:57-92: BFloat16, Float16, Float32, Float64, Int64..Int8, UInt64..UInt8
    L = _lib.lib()
    sizes = [L.btm_dtype_size(i) for i in range(13)]
    assert sizes == [2, 2, 4, 8, 8, 4, 2, 1, 8, 4, 2, 1, 1]
    assert L.btm_dtype_size(13) == 0 and L.btm_dtype_size(-1) == 0


def test_argument_errors_precede_device_work():
    L = _lib.lib()
    # unsupported dtype -> NotImplemented-class status, with a message
    rc = L.btm_gemm(0, None, _lib.I32, 4, 4, 4, None, 4, None, 4, None, 4)
    assert rc == _lib.ERR_UNSUPPORTED and b"dtype" in L.btm_last_error_string()
    rc = L.btm_gemm(0, None, _lib.F16, -1, 4, 4, None, 4, None, 4, None, 4)
    assert rc == _lib.ERR_INVALID
    rc = L.btm_gemm(0, None, _lib.F16, 4, 4, 4, ctypes.c_void_p(16), 2, ctypes.c_void_p(16), 4, ctypes.c_void_p(16), 4)
    assert rc == _lib.ERR_INVALID and b"leading dimension" in L.btm_last_error_string()
    rc = L.btm_int4_matmul(0, None, 1, 16, 100, 128, None, None, None, None)
    assert rc == _lib.ERR_INVALID
    rc = L.btm_bmm(0, None, _lib.F32, 1, 4, 4, 4, None, 16, None, 16, None, 16)
    assert rc == _lib.ERR_UNSUPPORTED
    # fused epilogue: an unknown activation code is refused before any device work
    p = ctypes.c_void_p(16)
    rc = L.btm_gemm_bias_act(0, None, _lib.F16, 4, 4, 4, p, 4, p, 4, None, 7, p, 4)
    assert rc == _lib.ERR_INVALID and b"activation" in L.btm_last_error_string()
    rc = L.btm_gemm_bias_act(0, None, _lib.I32, 4, 4, 4, p, 4, p, 4, None, 1, p, 4)
    assert rc == _lib.ERR_UNSUPPORTED


def test_no_cpu_fallback_without_device():
    import torch
    if torch.cuda.is_available():
        return
    L = _lib.lib()
    assert L.btm_init(0) in (_lib.ERR_CUDA, _lib.ERR_INVALID)
    assert L.btm_last_error_string() != b""
