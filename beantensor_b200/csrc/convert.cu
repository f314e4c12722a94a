// Format producers on either side of the matmul path (HBM-bound element-wise kernels):
//   - dtype conversion fp32 <-> fp16 / bf16 with round-to-nearest-even, the rounding the reference's CUDA
//     conversion uses (Tensor/TensorOps.cu:59-84); the reference covers fp32 <-> bf16 only (:337-345);
//   - int4 group quantiser: fp16 weights [N,K] -> packed nibbles [N,K/2] + one fp16 scale per group, the
//     producer of the format btm_int4_matmul consumes.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "btm_internal.h"

namespace btm {

template <typename S, typename D>
__device__ __forceinline__ D cvt(S x);
template <> __device__ __forceinline__ __half cvt<float, __half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt<float, __nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ float cvt<__half, float>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float cvt<__nv_bfloat16, float>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt<__half, __nv_bfloat16>(__half x) { return __float2bfloat16_rn(__half2float(x)); }
template <> __device__ __forceinline__ __half cvt<__nv_bfloat16, __half>(__nv_bfloat16 x) { return __float2half_rn(__bfloat162float(x)); }

template <typename S, typename D>
__global__ void convert_kernel(const S *__restrict__ src, D *__restrict__ dst, long long n)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = cvt<S, D>(src[i]);
}

template <typename S, typename D>
static int run_convert(cudaStream_t st, const void *src, void *dst, long long n)
{
    const int block = 256;
    long long g = (n + block - 1) / block;
    if (g > 148LL * 32) g = 148LL * 32;
    convert_kernel<S, D><<<(unsigned)g, block, 0, st>>>((const S *)src, (D *)dst, n);
    return check_cuda(cudaGetLastError(), "convert launch");
}

int launch_convert(cudaStream_t st, int src_dtype, int dst_dtype, long long n, const void *src, void *dst)
{
    if (n == 0) return BTM_OK;
    if (src_dtype == BTM_F32 && dst_dtype == BTM_F16) return run_convert<float, __half>(st, src, dst, n);
    if (src_dtype == BTM_F32 && dst_dtype == BTM_BF16) return run_convert<float, __nv_bfloat16>(st, src, dst, n);
    if (src_dtype == BTM_F16 && dst_dtype == BTM_F32) return run_convert<__half, float>(st, src, dst, n);
    if (src_dtype == BTM_BF16 && dst_dtype == BTM_F32) return run_convert<__nv_bfloat16, float>(st, src, dst, n);
    if (src_dtype == BTM_F16 && dst_dtype == BTM_BF16) return run_convert<__half, __nv_bfloat16>(st, src, dst, n);
    if (src_dtype == BTM_BF16 && dst_dtype == BTM_F16) return run_convert<__nv_bfloat16, __half>(st, src, dst, n);
    return set_error(BTM_ERR_UNSUPPORTED, "convert: %d -> %d is not supported (Float32, Float16, BFloat16 only)", src_dtype, dst_dtype);
}

// One warp per (row, group): amax over the group, scale = f16_rne(amax / 7) (1 when the group is all zero),
// q = clamp(rint(w / scale), -8, 7); nibbles packed two per byte, even k in bits 0-3.
__global__ void int4_quantize_kernel(int N, int K, int group, const __half *__restrict__ w, uint8_t *__restrict__ packed,
                                     __half *__restrict__ scales)
{
    const int G = K / group;
    const long long warp_id = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const long long total = (long long)N * G;
    if (warp_id >= total) return;
    const long long n = warp_id / G;
    const int gi = (int)(warp_id - n * G);
    const __half *src = w + n * K + (long long)gi * group;
    float amax = 0.f;
    for (int k = lane; k < group; k += 32) amax = fmaxf(amax, fabsf(__half2float(src[k])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    __half sh = __float2half_rn(__fdiv_rn(amax, 7.0f));
    if (__half2float(sh) == 0.f) sh = __float2half_rn(1.0f);
    const float s = __half2float(sh);
    if (lane == 0) scales[n * G + gi] = sh;
    uint8_t *dst = packed + n * (K / 2) + (long long)gi * (group / 2);
    for (int b = lane; b < group / 2; b += 32) {
        const float q0 = fminf(fmaxf(rintf(__fdiv_rn(__half2float(src[2 * b]), s)), -8.f), 7.f);
        const float q1 = fminf(fmaxf(rintf(__fdiv_rn(__half2float(src[2 * b + 1]), s)), -8.f), 7.f);
        dst[b] = (uint8_t)(((int)q0 & 0xF) | (((int)q1 & 0xF) << 4));
    }
}

int launch_int4_quantize(cudaStream_t st, int N, int K, int group, const void *w, void *packed, void *scales)
{
    const long long warps = (long long)N * (K / group);
    if (warps == 0) return BTM_OK;
    const int block = 256;
    const long long grid = (warps * 32 + block - 1) / block;
    if (grid > 0x7FFFFFFFLL) return set_error(BTM_ERR_UNSUPPORTED, "int4 quantise: too many groups");
    int4_quantize_kernel<<<(unsigned)grid, block, 0, st>>>(N, K, group, (const __half *)w, (uint8_t *)packed, (__half *)scales);
    return check_cuda(cudaGetLastError(), "int4 quantise launch");
}

} // namespace btm
