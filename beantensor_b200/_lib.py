"""ctypes binding of libbtm.so (the C ABI declared in include/btm.h).

The library is the product; this module only loads it and declares argument types. There is
no Python or CPU fallback: if the shared object is missing, `lib()` raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("BTM_LIB") or os.path.join(HERE, "libbtm.so")  # BTM_LIB: load another build of the library

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_OOM, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT = range(7)
BF16, F16, F32, F64, I64, I32, I16, I8, U64, U32, U16, U8, INT4X2 = range(13)  # Tensor/Dtypes.h:57-70 + appended int4

_i, _i64, _vp, _sz = C.c_int, C.c_int64, C.c_void_p, C.c_size_t

SIGNATURES = {
    "btm_dtype_size": (_sz, [_i]),
    "btm_version": (_i, []),
    "btm_last_error_string": (C.c_char_p, []),
    "btm_debug_set": (_i, [C.c_char_p, C.c_longlong]),
    "btm_init": (_i, [_i]),
    "btm_check_device_status": (_i, [_i, _vp]),
    "btm_gemm": (_i, [_i, _vp, _i, _i, _i, _i, _vp, _i64, _vp, _i64, _vp, _i64]),
    "btm_gemm_bias_act": (_i, [_i, _vp, _i, _i, _i, _i, _vp, _i64, _vp, _i64, _vp, _i, _vp, _i64]),
    "btm_gemm_bt": (_i, [_i, _vp, _i, _i, _i, _i, _vp, _i64, _vp, _i64, _vp, _i64]),
    "btm_gemm_strided": (_i, [_i, _vp, _i, _i, _i, _i, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64]),
    "btm_gemm_f32_workspace_bytes": (_sz, [_i, _i, _i]),
    "btm_gemm_f32_ws": (_i, [_i, _vp, _i, _i, _i, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _sz]),
    "btm_gemm_f32_static": (_i, [_i, _vp, _i, _i, _i, _vp, _i64, _vp, _i64, _vp, _i64]),
    "btm_bmm": (_i, [_i, _vp, _i, _i, _i, _i, _i, _vp, _i64, _vp, _i64, _vp, _i64]),
    "btm_int4_matmul": (_i, [_i, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "btm_int4_dequant": (_i, [_i, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "btm_int4_quantize": (_i, [_i, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "btm_convert": (_i, [_i, _vp, _i, _i, _i64, _vp, _vp]),
    "btm_int4_unpack": (_i, [_i, _vp, _i, _i, _vp, _vp]),
    "btm_gemm_nshard": (_i, [_i, _vp, _i, _i, _i, _i, _vp, _i64, _vp, _i64, C.POINTER(_vp), _i64, _i, _i]),
    "btm_gemm_nshard_mc": (_i, [_i, _vp, _i, _i, _i, _i, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i, _i]),
    "btm_mc_supported": (_i, [_i]),
    "btm_mc_create": (_i, [_i, _i, _sz, C.POINTER(_vp), C.POINTER(_i)]),
    "btm_mc_import": (_i, [_i, _i, _sz, _i, C.POINTER(_vp)]),
    "btm_mc_add_device": (_i, [_vp]),
    "btm_mc_bind": (_i, [_vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "btm_mc_release": (_i, [_vp]),
    "btm_replicate_rows": (_i, [_i, _vp, C.POINTER(_vp), _i, _i, _sz, _sz]),
    "btm_ipc_alloc": (_i, [_i, _sz, C.POINTER(_vp), C.c_char_p]),
    "btm_ipc_open": (_i, [_i, C.c_char_p, C.POINTER(_vp)]),
    "btm_ipc_close": (_i, [_i, _vp]),
    "btm_ipc_free": (_i, [_i, _vp]),
}

_lib = None


def lib() -> C.CDLL:
    """Load libbtm.so. Raises if it has not been built (python -m beantensor_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m beantensor_b200.build`. "
                "There is no fallback path; the CUDA library is the implementation.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return lib().btm_last_error_string().decode("utf-8", "replace")
