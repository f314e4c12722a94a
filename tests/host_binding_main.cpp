// Compiled and run by tests/test_host_binding.py: exercises the C++ binding's guards and the
// status -> exception mapping without touching a GPU.
#include <cstdio>
#include <cstring>

#include "../beantensor_b200/host/MatMulOps.h"

using namespace BeanTensor::Tensors::detail;

static btm_tensor_view view(int dtype, int device, uint64_t r, uint64_t c)
{
    btm_tensor_view v;
    std::memset(&v, 0, sizeof(v));
    v.data = reinterpret_cast<void *>(0x1000);
    v.dtype = dtype;
    v.device = device;
    v.ndim = 2;
    v.shape[0] = r;
    v.shape[1] = c;
    v.strides[0] = c;
    v.strides[1] = 1;
    return v;
}

int main()
{
    int passed = 0;
    {   // CPU tensor -> std::invalid_argument, as the reference's guards do
        auto a = view(BTM_F16, 0, 4, 4), b = view(BTM_F16, 0, 4, 4), o = view(BTM_F16, 0, 4, 4);
        try { matmul_gpu(a, b, o); } catch (const std::invalid_argument &) { ++passed; }
    }
    {   // shape mismatch
        auto a = view(BTM_F16, 1, 4, 5), b = view(BTM_F16, 1, 4, 4), o = view(BTM_F16, 1, 4, 4);
        try { matmul_gpu(a, b, o); } catch (const std::invalid_argument &) { ++passed; }
    }
    {   // unsupported dtype comes back from the C ABI as NotImplemented
        auto a = view(BTM_I32, 1, 4, 4), b = view(BTM_I32, 1, 4, 4), o = view(BTM_I32, 1, 4, 4);
        try { matmul_gpu(a, b, o); } catch (const BeanTensor::ErrorHandling::NotImplemented &) { ++passed; }
    }
    {   // status mapping
        try { btm_raise(BTM_ERR_OOM); } catch (const std::bad_alloc &) { ++passed; }
        try { btm_raise(BTM_ERR_CUDA); } catch (const std::runtime_error &) { ++passed; }
        btm_raise(BTM_OK);
    }
    {   // fused epilogue: a bias of the wrong length is refused by the binding's own guard
        auto a = view(BTM_F16, 1, 4, 4), b = view(BTM_F16, 1, 4, 4), o = view(BTM_F16, 1, 4, 4);
        btm_tensor_view bias;
        std::memset(&bias, 0, sizeof(bias));
        bias.data = reinterpret_cast<void *>(0x1000);
        bias.dtype = BTM_F16;
        bias.device = 1;
        bias.ndim = 1;
        bias.shape[0] = 5;
        bias.strides[0] = 1;
        try { matmul_bias_act_gpu(a, b, &bias, true, o); } catch (const std::invalid_argument &) { ++passed; }
    }
    std::printf("passed=%d\n", passed);
    return passed == 6 ? 0 : 1;
}
