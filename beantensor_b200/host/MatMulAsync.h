// The reference-style asynchronous form of the matmul operators, and the user-level Ops::matmul.
//
// The reference's GPU operators do four things (Tensor/TensorOps.cu:89-93,203-207): check that the tensor is on the
// GPU, sync() it (wait for work queued on it earlier), hand a worker to the process-wide thread pool with High
// priority (Helper/Threads/CPUThreading.h:73-83), and attach the worker's future to the output tensor
// (Tensor::give_future, Tensor/Tensor.h:77-100); an exception thrown inside the worker surfaces at the next sync().
// The functions here are that pattern for the matmul family, written against two small concepts instead of the
// reference's classes so that they compile with or without the reference tree:
//   Pool    anything with  std::future<void> submit(F&&, Priority)      (ThreadPool of CPUThreading.h fits)
//   views   btm_tensor_view, the POD mirror of the Tensor fields the path reads
// Inside the reference tree the maintainer's detail::matmul_gpu(const Tensor&, const Tensor&, Tensor&) is
//   out.give_future(matmul_gpu_async(Threading::get_cpu_thread_pool(), Threading::ThreadPriority::High,
//                                    view_of(a), view_of(b), view_of(out)));
// after a.sync(); b.sync(); out.sync();
#pragma once
#include <future>
#include <utility>

#include "MatMulOps.h"

namespace BeanTensor::Tensors::detail {

// Guards run on the caller's thread (as the reference's device check does, TensorOps.cu:90); the product is enqueued
// by a pool worker. The views are captured by value: the caller's Tensor objects may move while the worker waits.
template <class Pool, class Priority>
std::shared_future<void> matmul_gpu_async(Pool &pool, Priority prio, btm_tensor_view a, btm_tensor_view b, btm_tensor_view out,
                                          void *stream = nullptr)
{
    if (out.device != 1) throw std::invalid_argument("Tensor is not on the GPU"); // TensorOps.cu:90
    return pool.submit([a, b, out, stream]() mutable { matmul_gpu(a, b, out, stream); }, prio).share();
}

template <class Pool, class Priority>
std::shared_future<void> bmm_gpu_async(Pool &pool, Priority prio, btm_tensor_view a, btm_tensor_view b, btm_tensor_view out,
                                       void *stream = nullptr)
{
    if (out.device != 1) throw std::invalid_argument("Tensor is not on the GPU");
    return pool.submit([a, b, out, stream]() mutable { bmm_gpu(a, b, out, stream); }, prio).share();
}

template <class Pool, class Priority>
std::shared_future<void> matmul_int4_gpu_async(Pool &pool, Priority prio, btm_tensor_view act, btm_tensor_view w_packed,
                                               btm_tensor_view scales, btm_tensor_view out, uint32_t group = 128, void *stream = nullptr)
{
    if (out.device != 1) throw std::invalid_argument("Tensor is not on the GPU");
    return pool.submit([act, w_packed, scales, out, group, stream]() mutable { matmul_int4_gpu(act, w_packed, scales, out, group, stream); }, prio)
        .share();
}

// Placement of a sharded operand: every rank holds rows [row0, row0 + rows) of a row-major [*, cols] matrix in its own
// copy `copies[rank]` and sends them to the same rows of every other rank's copy (peer-mapped views). The multi-GPU
// counterpart of the reference's move_gpu_to_gpu (Tensor/TensorOps.cu:282-313), which copies a whole tensor to one GPU.
inline void replicate_rows_gpu(const btm_tensor_view *copies, int rank, int nranks, uint64_t row0, uint64_t rows, void *stream = nullptr)
{
    if (!copies || nranks < 1 || rank < 0 || rank >= nranks) throw std::invalid_argument("replicate_rows_gpu: bad rank arguments");
    const btm_tensor_view &mine = copies[rank];
    btm_require_gpu_rowmajor(mine, 2, "replicate_rows_gpu");
    if (row0 + rows > mine.shape[0] || (mine.shape[0] > 1 && mine.strides[0] != mine.shape[1]))
        throw std::invalid_argument("replicate_rows_gpu: rows out of range or matrix not dense");
    void *bases[8];
    if (nranks > 8) throw std::invalid_argument("replicate_rows_gpu: at most 8 ranks");
    for (int r = 0; r < nranks; ++r) bases[r] = const_cast<void *>(btm_base(copies[r]));
    const size_t es = btm_dtype_size(mine.dtype);
    btm_raise(btm_replicate_rows(mine.gpu_id, stream, bases, rank, nranks, (size_t)(row0 * mine.shape[1]) * es, (size_t)(rows * mine.shape[1]) * es));
}

} // namespace BeanTensor::Tensors::detail

namespace BeanTensor::Ops {

// User-level product in the style of the reference's Ops::add sketch (Ops/Elementwise/Add/Add.h:28-73): checks the
// operands, makes the result tensor, dispatches by rank (2: matmul, 3: batched matmul) and returns it. `make_out`
// stands where the sketch calls Tensors::make_tensor(shape, ndims, dtype, device, requires_grad): it receives the
// result's shape, rank, dtype ordinal and GPU ordinal and returns a view of freshly allocated device memory.
template <class MakeOut>
[[nodiscard]] btm_tensor_view matmul(const btm_tensor_view &a, const btm_tensor_view &b, MakeOut &&make_out, void *stream = nullptr)
{
    namespace d = BeanTensor::Tensors::detail;
    if (a.device != b.device || a.gpu_id != b.gpu_id) throw std::invalid_argument("matmul: operands live on different devices"); // assert(t1.device == t2.device), Add.h:30
    if (a.dtype != b.dtype) throw std::invalid_argument("matmul: dtypes differ");
    if (a.ndim != b.ndim || (a.ndim != 2 && a.ndim != 3)) throw std::invalid_argument("matmul: operands must both have rank 2 or rank 3");
    uint64_t shape[8] = {0};
    if (a.ndim == 2) {
        if (a.shape[1] != b.shape[0]) throw std::invalid_argument("matmul: inner dimensions differ");
        shape[0] = a.shape[0];
        shape[1] = b.shape[1];
    } else {
        if (a.shape[0] != b.shape[0] || a.shape[2] != b.shape[1]) throw std::invalid_argument("matmul: batch or inner dimensions differ");
        shape[0] = a.shape[0];
        shape[1] = a.shape[1];
        shape[2] = b.shape[2];
    }
    btm_tensor_view out = make_out(shape, a.ndim, a.dtype, a.gpu_id);
    if (a.ndim == 2) d::matmul_gpu(a, b, out, stream);
    else d::bmm_gpu(a, b, out, stream);
    return out;
}

} // namespace BeanTensor::Ops
