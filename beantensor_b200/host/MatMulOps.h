// C++23 binding of libbtm.so in the style of the reference's GPU operator boundary
// (namespace BeanTensor::Tensors::detail, Tensor/TensorOps.h:15-65): free functions that guard
// the device, enqueue the work and leave the result in a pre-allocated tensor, raising the
// reference's exception types (Errors/Logic.h:13-59) on failure.
//
// The functions take btm_tensor_view, a POD mirror of the Tensor fields the path reads
// (Tensor/Tensor.h:173-201). Inside the reference tree a maintainer fills it from a Tensor in a
// friend function and defines BT_HAVE_REFERENCE_ERRORS so that the
// exception types come from Errors/Logic.h instead of the stand-ins below.
#pragma once
#include <cstdint>
#include <new>
#include <stdexcept>
#include <string>

#include "../../include/btm.h"

#if defined(BT_HAVE_REFERENCE_ERRORS)
#include "Errors/Logic.h"
#else
namespace BeanTensor::ErrorHandling {
class NotImplemented : public std::logic_error {
public:
    NotImplemented() : std::logic_error("Function not yet implemented") {}
};
class OutOfMemory : public std::bad_alloc {
public:
    OutOfMemory() = default;
};
} // namespace BeanTensor::ErrorHandling
#endif

namespace BeanTensor::Tensors::detail {

// Status -> exception, the inverse of what a C ABI has to do to the reference's throw sites.
inline void btm_raise(int status)
{
    if (status == BTM_OK) return;
    const std::string msg = btm_last_error_string();
    switch (status) {
    case BTM_ERR_INVALID: throw std::invalid_argument(msg);                       // Tensor/TensorOps.cu:241,269
    case BTM_ERR_UNSUPPORTED: throw BeanTensor::ErrorHandling::NotImplemented();  // Errors/Logic.h:13-17
    case BTM_ERR_OOM: throw BeanTensor::ErrorHandling::OutOfMemory();             // Errors/Logic.h:22-25
    default: throw std::runtime_error(msg);                                       // "CUDA Error: ..." Errors/Logic.h:50-59
    }
}

inline void btm_require_gpu_rowmajor(const btm_tensor_view &t, int ndim, const char *name)
{
    if (t.device != 1) throw std::invalid_argument(std::string(name) + ": Tensor is not on the GPU"); // guard of TensorOps.cu:89-93
    if (t.ndim != ndim) throw std::invalid_argument(std::string(name) + ": wrong rank");
    if (t.shape[ndim - 1] > 1 && t.strides[ndim - 1] != 1)
        throw std::invalid_argument(std::string(name) + ": last dimension must be contiguous (row-major, Tensor.cpp:157-162)");
}

inline const void *btm_base(const btm_tensor_view &t)
{
    return static_cast<const char *>(t.data) + t.offset * btm_dtype_size(t.dtype);
}

// out[M,N] = act(a[M,K] . b[K,N] + bias[N]). Float16/BFloat16 (fp32 accumulate) or Float32 (3xTF32).
// `bias` may be null (none); `relu` applies max(x, 0) after the bias. The product, the reference's broadcast Add
// (Ops/Elementwise/Add/Add.h:28) and its Relu stub (Ops/Elementwise/Relu/Relu.h) in one kernel: out is written once.
inline void matmul_bias_act_gpu(const btm_tensor_view &a, const btm_tensor_view &b, const btm_tensor_view *bias, bool relu,
                                btm_tensor_view &out, void *stream = nullptr)
{
    btm_require_gpu_rowmajor(a, 2, "matmul_gpu(a)");
    btm_require_gpu_rowmajor(b, 2, "matmul_gpu(b)");
    btm_require_gpu_rowmajor(out, 2, "matmul_gpu(out)");
    if (a.dtype != b.dtype || a.dtype != out.dtype) throw std::invalid_argument("matmul_gpu: dtypes differ");
    if (a.gpu_id != b.gpu_id || a.gpu_id != out.gpu_id) throw std::invalid_argument("matmul_gpu: tensors live on different GPUs");
    if (a.shape[1] != b.shape[0] || out.shape[0] != a.shape[0] || out.shape[1] != b.shape[1])
        throw std::invalid_argument("matmul_gpu: shape mismatch");
    if (bias) {
        btm_require_gpu_rowmajor(*bias, 1, "matmul_gpu(bias)");
        if (bias->dtype != out.dtype || bias->gpu_id != out.gpu_id || bias->shape[0] != out.shape[1])
            throw std::invalid_argument("matmul_gpu: bias must be a [N] tensor of the output's dtype on the output's GPU");
    }
    const int M = (int)a.shape[0], K = (int)a.shape[1], N = (int)b.shape[1];
    const int64_t lda = M > 1 ? (int64_t)a.strides[0] : (K > 0 ? K : 1);
    const int64_t ldb = K > 1 ? (int64_t)b.strides[0] : (N > 0 ? N : 1);
    const int64_t ldc = M > 1 ? (int64_t)out.strides[0] : (N > 0 ? N : 1);
    btm_raise(btm_gemm_bias_act(a.gpu_id, stream, a.dtype, M, N, K, btm_base(a), lda, btm_base(b), ldb, bias ? btm_base(*bias) : nullptr,
                                relu ? BTM_ACT_RELU : BTM_ACT_NONE, const_cast<void *>(btm_base(out)), ldc));
}

// Operands may be any 2-D view (Tensor::strides, Tensor/Tensor.h:173-195): row-major, transposed or strided.
inline void btm_require_gpu_2d(const btm_tensor_view &t, const char *name)
{
    if (t.device != 1) throw std::invalid_argument(std::string(name) + ": Tensor is not on the GPU"); // guard of TensorOps.cu:89-93
    if (t.ndim != 2) throw std::invalid_argument(std::string(name) + ": wrong rank");
}

// out[M,N] = a[M,K] . b[K,N]. Float16/BFloat16 (fp32 accumulate) or Float32 (3xTF32). a and b may be transposed or
// strided views (no copy is made); out is row-major.
inline void matmul_gpu(const btm_tensor_view &a, const btm_tensor_view &b, btm_tensor_view &out, void *stream = nullptr)
{
    btm_require_gpu_2d(a, "matmul_gpu(a)");
    btm_require_gpu_2d(b, "matmul_gpu(b)");
    btm_require_gpu_rowmajor(out, 2, "matmul_gpu(out)");
    if (a.dtype != b.dtype || a.dtype != out.dtype) throw std::invalid_argument("matmul_gpu: dtypes differ");
    if (a.gpu_id != b.gpu_id || a.gpu_id != out.gpu_id) throw std::invalid_argument("matmul_gpu: tensors live on different GPUs");
    if (a.shape[1] != b.shape[0] || out.shape[0] != a.shape[0] || out.shape[1] != b.shape[1])
        throw std::invalid_argument("matmul_gpu: shape mismatch");
    const int M = (int)a.shape[0], K = (int)a.shape[1], N = (int)b.shape[1];
    const int64_t ldc = M > 1 ? (int64_t)out.strides[0] : (N > 0 ? N : 1);
    btm_raise(btm_gemm_strided(a.gpu_id, stream, a.dtype, M, N, K, btm_base(a), (int64_t)a.strides[0], (int64_t)a.strides[1], btm_base(b),
                               (int64_t)b.strides[0], (int64_t)b.strides[1], const_cast<void *>(btm_base(out)), ldc));
}

// out[b] = a[b] . b[b]; dense row-major matrices with a batch stride.
inline void bmm_gpu(const btm_tensor_view &a, const btm_tensor_view &b, btm_tensor_view &out, void *stream = nullptr)
{
    btm_require_gpu_rowmajor(a, 3, "bmm_gpu(a)");
    btm_require_gpu_rowmajor(b, 3, "bmm_gpu(b)");
    btm_require_gpu_rowmajor(out, 3, "bmm_gpu(out)");
    if (a.dtype != b.dtype || a.dtype != out.dtype) throw std::invalid_argument("bmm_gpu: dtypes differ");
    if (a.shape[0] != b.shape[0] || a.shape[0] != out.shape[0] || a.shape[2] != b.shape[1] || out.shape[1] != a.shape[1] ||
        out.shape[2] != b.shape[2])
        throw std::invalid_argument("bmm_gpu: shape mismatch");
    const int B = (int)a.shape[0], M = (int)a.shape[1], K = (int)a.shape[2], N = (int)b.shape[2];
    if ((M > 1 && a.strides[1] != (uint64_t)K) || (K > 1 && b.strides[1] != (uint64_t)N) || (M > 1 && out.strides[1] != (uint64_t)N))
        throw std::invalid_argument("bmm_gpu: each matrix must be dense row-major");
    btm_raise(btm_bmm(a.gpu_id, stream, a.dtype, B, M, N, K, btm_base(a), (int64_t)a.strides[0], btm_base(b), (int64_t)b.strides[0],
                      const_cast<void *>(btm_base(out)), (int64_t)out.strides[0]));
}

// out[M,N] (Float16) = act[M,K] (Float16) . dequant(w_packed[N,K/2], scales[N,K/group])^T
inline void matmul_int4_gpu(const btm_tensor_view &act, const btm_tensor_view &w_packed, const btm_tensor_view &scales,
                            btm_tensor_view &out, uint32_t group = 128, void *stream = nullptr)
{
    btm_require_gpu_rowmajor(act, 2, "matmul_int4_gpu(act)");
    btm_require_gpu_rowmajor(w_packed, 2, "matmul_int4_gpu(w)");
    btm_require_gpu_rowmajor(scales, 2, "matmul_int4_gpu(scales)");
    btm_require_gpu_rowmajor(out, 2, "matmul_int4_gpu(out)");
    if (act.dtype != BTM_F16 || scales.dtype != BTM_F16 || out.dtype != BTM_F16 || w_packed.dtype != BTM_INT4X2)
        throw std::invalid_argument("matmul_int4_gpu: expected Float16 activations/scales/output and packed int4 weights");
    const int M = (int)act.shape[0], K = (int)act.shape[1], N = (int)w_packed.shape[0];
    if (group == 0 || w_packed.shape[1] * 2 != (uint64_t)K || scales.shape[0] != (uint64_t)N || scales.shape[1] * group != (uint64_t)K ||
        out.shape[0] != (uint64_t)M || out.shape[1] != (uint64_t)N)
        throw std::invalid_argument("matmul_int4_gpu: shape mismatch");
    btm_raise(btm_int4_matmul(act.gpu_id, stream, M, N, K, (int)group, btm_base(act), btm_base(w_packed), btm_base(scales),
                              const_cast<void *>(btm_base(out))));
}

} // namespace BeanTensor::Tensors::detail
