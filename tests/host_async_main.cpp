// Compiled and run by tests/test_host_binding.py. Exercises the reference-style asynchronous operators: workers on a
// thread pool, futures joined by the caller, exceptions surfacing at future.get(). With BT_HAVE_REFERENCE_POOL the pool
// is the reference's own ThreadPool (Helper/Threads/CPUThreading.h, header-only, taken from the reference tree by
// include path); otherwise a stand-in with the same submit() signature. With the argument "gpu" the workers run real
// products on cuda:0 and the results are compared with the CPU checker (oracle/libbtm_oracle.so).
#include <cuda_runtime_api.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <thread>
#include <vector>

#include "../beantensor_b200/host/MatMulAsync.h"

#if defined(BT_HAVE_REFERENCE_POOL)
#include "Helper/Threads/CPUThreading.h"
using Pool = BeanTensor::Threading::ThreadPool;
using Priority = BeanTensor::Threading::ThreadPriority;
static Pool &the_pool() { return BeanTensor::Threading::get_cpu_thread_pool(); }
static const char *pool_name = "reference ThreadPool";
#else
enum class Priority { Low = 1, Normal = 2, High = 3 };
struct Pool { // one thread per task: the smallest thing with the reference pool's submit() signature
    template <typename F>
    std::future<void> submit(F &&f, Priority = Priority::Normal)
    {
        std::packaged_task<void()> task(std::forward<F>(f));
        std::future<void> fut = task.get_future();
        std::thread(std::move(task)).detach();
        return fut;
    }
};
static Pool &the_pool() { static Pool p; return p; }
static const char *pool_name = "stand-in pool";
#endif

extern "C" int btmo_gemm(int dtype, int64_t M, int64_t N, int64_t K, const void *A, int64_t lda, const void *B, int64_t ldb, double *C,
                         int64_t ldc, int threads);

using namespace BeanTensor::Tensors::detail;

static btm_tensor_view view2(void *data, int dtype, int device, uint64_t r, uint64_t c)
{
    btm_tensor_view v;
    std::memset(&v, 0, sizeof(v));
    v.data = data;
    v.dtype = dtype;
    v.device = device;
    v.ndim = 2;
    v.shape[0] = r;
    v.shape[1] = c;
    v.strides[0] = c;
    v.strides[1] = 1;
    return v;
}

int main(int argc, char **argv)
{
    const bool gpu = argc > 1 && !std::strcmp(argv[1], "gpu");
    int passed = 0;
    Pool &pool = the_pool();
    void *fake = reinterpret_cast<void *>(0x1000);
    {   // a bad shape is found by the worker, travels in the future and is thrown at get(), as at Tensor::sync()
        auto a = view2(fake, BTM_F16, 1, 4, 5), b = view2(fake, BTM_F16, 1, 4, 4), o = view2(fake, BTM_F16, 1, 4, 4);
        auto fut = matmul_gpu_async(pool, Priority::High, a, b, o);
        try { fut.get(); } catch (const std::invalid_argument &) { ++passed; }
    }
    {   // the device guard runs on the caller's thread, before anything is submitted
        auto a = view2(fake, BTM_F16, 1, 4, 4), o = view2(fake, BTM_F16, 0, 4, 4);
        try { (void)matmul_gpu_async(pool, Priority::High, a, a, o); } catch (const std::invalid_argument &) { ++passed; }
    }
    {   // an unsupported dtype comes back from the C ABI inside the worker as NotImplemented
        auto a = view2(fake, BTM_I32, 1, 4, 4), o = view2(fake, BTM_I32, 1, 4, 4);
        auto fut = matmul_gpu_async(pool, Priority::High, a, a, o);
        try { fut.get(); } catch (const BeanTensor::ErrorHandling::NotImplemented &) { ++passed; }
    }
    {   // Ops::matmul: rank and shape checks happen before the result is made
        auto a = view2(fake, BTM_F16, 1, 4, 5), b = view2(fake, BTM_F16, 1, 6, 4);
        bool made = false;
        try {
            (void)BeanTensor::Ops::matmul(a, b, [&](const uint64_t *, int, int, int) { made = true; return btm_tensor_view{}; });
        } catch (const std::invalid_argument &) { if (!made) ++passed; }
    }
    if (gpu) {
        // Four tensors, four workers, one product each on cuda:0 (null stream, as the reference does), joined by futures.
        const int n = 256, jobs = 4;
        std::vector<std::vector<float>> A(jobs), B(jobs), C(jobs);
        std::vector<float *> dA(jobs), dB(jobs), dC(jobs);
        std::vector<std::shared_future<void>> futs;
        for (int j = 0; j < jobs; ++j) {
            A[j].resize(n * n); B[j].resize(n * n); C[j].assign(n * n, -1.f);
            for (int i = 0; i < n * n; ++i) {
                A[j][i] = (float)((i * 37 + j * 11) % 201 - 100) / 100.f;
                B[j][i] = (float)((i * 53 + j * 7) % 197 - 98) / 98.f;
            }
            if (cudaMalloc((void **)&dA[j], n * n * 4) || cudaMalloc((void **)&dB[j], n * n * 4) || cudaMalloc((void **)&dC[j], n * n * 4)) return 2;
            cudaMemcpy(dA[j], A[j].data(), n * n * 4, cudaMemcpyHostToDevice);
            cudaMemcpy(dB[j], B[j].data(), n * n * 4, cudaMemcpyHostToDevice);
        }
        for (int j = 0; j < jobs; ++j)
            futs.push_back(matmul_gpu_async(pool, Priority::High, view2(dA[j], BTM_F32, 1, n, n), view2(dB[j], BTM_F32, 1, n, n), view2(dC[j], BTM_F32, 1, n, n)));
        for (auto &f : futs) f.get();
        cudaDeviceSynchronize();
        int good = 0;
        for (int j = 0; j < jobs; ++j) {
            cudaMemcpy(C[j].data(), dC[j], n * n * 4, cudaMemcpyDeviceToHost);
            std::vector<double> ref(n * n);
            btmo_gemm(2 /* Float32 */, n, n, n, A[j].data(), n, B[j].data(), n, ref.data(), n, 4);
            double num = 0, den = 0;
            for (int i = 0; i < n * n; ++i) { num += (C[j][i] - ref[i]) * (C[j][i] - ref[i]); den += ref[i] * ref[i]; }
            if (std::sqrt(num / den) <= 1e-5) ++good;
        }
        if (good == jobs) ++passed;
        // Ops::matmul with a real allocator: the result tensor is made by the callback and filled by the product
        {
            float *dOut = nullptr;
            auto out = BeanTensor::Ops::matmul(view2(dA[0], BTM_F32, 1, n, n), view2(dB[0], BTM_F32, 1, n, n),
                                               [&](const uint64_t *shape, int ndim, int dtype, int gpu_id) {
                                                   cudaMalloc((void **)&dOut, shape[0] * shape[1] * 4);
                                                   auto v = view2(dOut, dtype, 1, shape[0], shape[1]);
                                                   v.gpu_id = gpu_id;
                                                   (void)ndim;
                                                   return v;
                                               });
            cudaDeviceSynchronize();
            std::vector<float> got(n * n);
            cudaMemcpy(got.data(), out.data, n * n * 4, cudaMemcpyDeviceToHost);
            if (std::memcmp(got.data(), C[0].data(), n * n * 4) == 0) ++passed; // same inputs, same kernel: same bits
            cudaFree(dOut);
        }
        for (int j = 0; j < jobs; ++j) { cudaFree(dA[j]); cudaFree(dB[j]); cudaFree(dC[j]); }
    }
    std::printf("pool=%s passed=%d\n", pool_name, passed);
    return passed == (gpu ? 6 : 4) ? 0 : 1;
}
