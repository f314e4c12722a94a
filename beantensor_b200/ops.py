"""Host-side mirror of the reference's GPU operator boundary for the matmul path.

The reference declares its GPU operators as free functions `detail::*_gpu(Tensor&, ...)`
(Tensor/TensorOps.h:15-65) that check the device, then enqueue work and leave the result in a
pre-allocated tensor. The functions here have the names and argument meaning a
`matmul_gpu` / `bmm_gpu` / `matmul_int4_gpu` family added beside them would have; torch
tensors stand in for BeanTensor's Tensor (torch is used for device memory and streams only —
every product is computed by libbtm.so).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .errors import GPUTaskOnCPUBuild, raise_for_status

_DT = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}


def _LIB():
    return _lib._lib or _lib.lib()


def _require_gpu(*tensors: torch.Tensor) -> int:
    if not torch.cuda.is_available():
        raise GPUTaskOnCPUBuild("GPU task cannot be run on CPU build")  # TensorOps.hpp:5-30
    dev = None
    for t in tensors:
        if t.device.type != "cuda":
            raise ValueError("Tensor is not on the GPU")  # guard of Tensor/TensorOps.cu:89-93
        if dev is None:
            dev = t.device.index
        elif t.device.index != dev:
            raise ValueError("Tensors live on different GPUs")
    return int(dev)


def _stream(dev: int | None = None) -> int:
    """The calling thread's current CUDA stream of `dev` as a raw handle (what the C ABI takes as void*)."""
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device() if dev is None else dev)


def _rowmajor(t: torch.Tensor, name: str) -> None:
    if t.stride(-1) != 1 and t.size(-1) > 1:
        raise ValueError(f"{name} must be row-major (last stride 1)")  # Tensor/Tensor.cpp:157-162


def init(device: int = 0) -> None:
    raise_for_status(_lib.lib().btm_init(device))


def check_device_status(device: int = 0) -> None:
    raise_for_status(_lib.lib().btm_check_device_status(device, _stream(device)))


def matmul_gpu(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
               relu: bool = False) -> None:
    """out[M,N] = a[M,K] . b[K,N]; fp16/bf16 (fp32 accumulate) or fp32 (3xTF32).

    With `bias` ([N], dtype of out) and/or `relu` the epilogue is fused: out = relu(a.b + bias), rounded once.
    """
    dev = _require_gpu(a, b, out)
    if bias is not None:
        if not bias.is_cuda or bias.device != out.device:
            raise ValueError("matmul_gpu: bias is not on the output's GPU")
        if bias.dim() != 1 or bias.shape[0] != out.shape[-1] or bias.dtype != out.dtype or not bias.is_contiguous():
            raise ValueError("matmul_gpu: bias must be a contiguous [N] tensor of the output's dtype")
    if a.dim() != 2 or b.dim() != 2 or out.dim() != 2:
        raise ValueError("matmul_gpu takes 2-D tensors")
    if a.dtype != b.dtype or a.dtype != out.dtype:
        raise ValueError("matmul_gpu: dtypes differ")
    if a.dtype not in _DT:
        from .errors import NotImplementedOp
        raise NotImplementedOp(f"matmul_gpu: dtype {a.dtype} is not supported")
    M, K = a.shape
    K2, N = b.shape
    if K != K2 or out.shape != (M, N):
        raise ValueError(f"matmul_gpu: shape mismatch {tuple(a.shape)} x {tuple(b.shape)} -> {tuple(out.shape)}")
    _rowmajor(out, "out")
    ldc = out.stride(0) if M > 1 else max(N, 1)
    a_row = a.stride(1) == 1 or K <= 1
    b_row = b.stride(1) == 1 or N <= 1
    if not (a_row and b_row):
        # Transposed or strided views (Tensor::strides, Tensor/Tensor.h:173-195) go through without a copy.
        if bias is not None or relu:
            raise ValueError("matmul_gpu: the fused epilogue takes row-major operands")
        rc = _LIB().btm_gemm_strided(dev, _stream(dev), _DT[a.dtype], M, N, K, a.data_ptr(), a.stride(0), a.stride(1),
                                     b.data_ptr(), b.stride(0), b.stride(1), out.data_ptr(), ldc)
        raise_for_status(rc)
        return
    lda = a.stride(0) if M > 1 else max(K, 1)
    ldb = b.stride(0) if K > 1 else max(N, 1)
    if bias is None and not relu:
        rc = _lib.lib().btm_gemm(dev, _stream(dev), _DT[a.dtype], M, N, K, a.data_ptr(), lda, b.data_ptr(), ldb,
                                 out.data_ptr(), ldc)
    else:
        rc = _lib.lib().btm_gemm_bias_act(dev, _stream(dev), _DT[a.dtype], M, N, K, a.data_ptr(), lda, b.data_ptr(), ldb,
                                          bias.data_ptr() if bias is not None else None, 1 if relu else 0,
                                          out.data_ptr(), ldc)
    raise_for_status(rc)


def bmm_gpu(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """out[b] = a[b] . b[b] for dense row-major 3-D tensors (fp16/bf16)."""
    dev = _require_gpu(a, b, out)
    if a.dim() != 3 or b.dim() != 3 or out.dim() != 3:
        raise ValueError("bmm_gpu takes 3-D tensors")
    if a.dtype != b.dtype or a.dtype != out.dtype:
        raise ValueError("bmm_gpu: dtypes differ")
    if a.dtype not in (torch.float16, torch.bfloat16):
        from .errors import NotImplementedOp
        raise NotImplementedOp(f"bmm_gpu: dtype {a.dtype} is not supported")
    B, M, K = a.shape
    B2, K2, N = b.shape
    if B != B2 or K != K2 or out.shape != (B, M, N):
        raise ValueError("bmm_gpu: shape mismatch")
    for t in (a, b, out):
        if not t[0].is_contiguous() if B > 0 else False:
            raise ValueError("bmm_gpu: each matrix must be dense row-major")
    sa = a.stride(0) if B > 1 else M * K
    sb = b.stride(0) if B > 1 else K * N
    sc = out.stride(0) if B > 1 else M * N
    rc = _lib.lib().btm_bmm(dev, _stream(dev), _DT[a.dtype], B, M, N, K, a.data_ptr(), sa, b.data_ptr(), sb,
                            out.data_ptr(), sc)
    raise_for_status(rc)


def matmul_int4_gpu(act: torch.Tensor, w_packed: torch.Tensor, scales: torch.Tensor, out: torch.Tensor,
                    group: int = 128) -> None:
    """out[M,N] (fp16) = act[M,K] (fp16) . dequant(w_packed[N,K/2], scales[N,K/group])^T."""
    # One pass over the operands: this call sits in front of a kernel of a few microseconds (a decoder calls it once
    # per layer and token), so the guards are written to cost little. Same checks as the other operators.
    dev = out.device.index
    f16 = torch.float16
    if not (act.is_cuda and w_packed.is_cuda and scales.is_cuda and out.is_cuda):
        _require_gpu(act, w_packed, scales, out)  # raises with the operator boundary's messages
    if act.device != out.device or w_packed.device != out.device or scales.device != out.device:
        raise ValueError("Tensors live on different GPUs")
    if act.dtype != f16 or scales.dtype != f16 or out.dtype != f16:
        raise ValueError("matmul_int4_gpu: activations, scales and output are Float16")
    if w_packed.dtype != torch.uint8:
        raise ValueError("matmul_int4_gpu: packed weights are bytes (two nibbles each)")
    M, K = act.shape
    N = w_packed.shape[0]
    if w_packed.shape != (N, K // 2) or scales.shape != (N, K // group if group else 0) or out.shape != (M, N):
        raise ValueError("matmul_int4_gpu: shape mismatch")
    if not (act.is_contiguous() and w_packed.is_contiguous() and scales.is_contiguous() and out.is_contiguous()):
        raise ValueError("matmul_int4_gpu: tensors must be contiguous")
    rc = _LIB().btm_int4_matmul(dev, torch._C._cuda_getCurrentRawStream(dev), M, N, K, group, act.data_ptr(), w_packed.data_ptr(),
                                scales.data_ptr(), out.data_ptr())
    if rc:
        raise_for_status(rc)


def dequant_int4_gpu(w_packed: torch.Tensor, scales: torch.Tensor, out: torch.Tensor, group: int = 128) -> None:
    dev = _require_gpu(w_packed, scales, out)
    N, K2 = w_packed.shape
    K = K2 * 2
    if out.shape != (N, K) or out.dtype != torch.float16 or scales.dtype != torch.float16:
        raise ValueError("dequant_int4_gpu: shape or dtype mismatch")
    rc = _lib.lib().btm_int4_dequant(dev, _stream(dev), N, K, group, w_packed.data_ptr(), scales.data_ptr(), out.data_ptr())
    raise_for_status(rc)


def unpack_int4_gpu(w_packed: torch.Tensor, out: torch.Tensor) -> None:
    dev = _require_gpu(w_packed, out)
    N, K2 = w_packed.shape
    if out.shape != (N, K2 * 2) or out.dtype != torch.int8:
        raise ValueError("unpack_int4_gpu: shape or dtype mismatch")
    rc = _lib.lib().btm_int4_unpack(dev, _stream(dev), N, K2 * 2, w_packed.data_ptr(), out.data_ptr())
    raise_for_status(rc)


def quantize_int4_gpu(w: torch.Tensor, w_packed: torch.Tensor, scales: torch.Tensor, group: int = 128) -> None:
    """fp16 weights [N,K] -> packed nibbles [N,K/2] + fp16 scales [N,K/group] (max-abs / 7 per group)."""
    dev = _require_gpu(w, w_packed, scales)
    N, K = w.shape
    if w.dtype != torch.float16 or scales.dtype != torch.float16 or w_packed.dtype != torch.uint8:
        raise ValueError("quantize_int4_gpu: Float16 weights and scales, byte output")
    if group <= 0 or K % group or w_packed.shape != (N, K // 2) or scales.shape != (N, K // group):
        raise ValueError("quantize_int4_gpu: shape mismatch")
    for t in (w, w_packed, scales):
        if not t.is_contiguous():
            raise ValueError("quantize_int4_gpu: tensors must be contiguous")
    rc = _lib.lib().btm_int4_quantize(dev, _stream(dev), N, K, group, w.data_ptr(), w_packed.data_ptr(), scales.data_ptr())
    raise_for_status(rc)


def convert_gpu(src: torch.Tensor, dst: torch.Tensor) -> None:
    """dst = dtype conversion of src (Float32 / Float16 / BFloat16, round to nearest even); the matmul-side
    counterpart of the reference's convert_gpu (Tensor/TensorOps.cu:315-365), out of place."""
    dev = _require_gpu(src, dst)
    if src.shape != dst.shape or not src.is_contiguous() or not dst.is_contiguous():
        raise ValueError("convert_gpu: shapes differ or tensors are not contiguous")
    if src.dtype not in _DT or dst.dtype not in _DT:
        from .errors import NotImplementedOp
        raise NotImplementedOp(f"convert_gpu: {src.dtype} -> {dst.dtype} is not supported")
    rc = _lib.lib().btm_convert(dev, _stream(dev), _DT[src.dtype], _DT[dst.dtype], src.numel(), src.data_ptr(), dst.data_ptr())
    raise_for_status(rc)


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """User-level wrapper in the style of the reference's Ops::add sketch
    (Ops/Elementwise/Add/Add.h:28-73): checks, allocates the result, dispatches by rank."""
    if a.dim() == 3:
        out = torch.empty((a.shape[0], a.shape[1], b.shape[2]), dtype=a.dtype, device=a.device)
        bmm_gpu(a, b, out)
        return out
    out = torch.empty((a.shape[0], b.shape[1]), dtype=a.dtype, device=a.device)
    matmul_gpu(a, b, out)
    return out
