// General CUDA-core matmul: the same contract as the tensor-core kernels (fp32 accumulation,
// round-to-nearest-even output) for shapes and pointers that TMA cannot address (row pitch or base not
// 16-byte aligned, K == 0) and for operands with arbitrary row and column strides. Any M, N, K and any alignment.
// 64 x 64 output tile per CTA, 16-deep k-slices through shared memory, 4 x 4 outputs per thread.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "btm_internal.h"

namespace btm {

template <int DT>
struct Elem;
template <>
struct Elem<BTM_F32> {
    using T = float;
    static __device__ __forceinline__ float load(const T *p) { return *p; }
    static __device__ __forceinline__ void store(T *p, float v) { *p = v; }
};
template <>
struct Elem<BTM_F16> {
    using T = __half;
    static __device__ __forceinline__ float load(const T *p) { return __half2float(*p); }
    static __device__ __forceinline__ void store(T *p, float v) { *p = __float2half_rn(v); }
};
template <>
struct Elem<BTM_BF16> {
    using T = __nv_bfloat16;
    static __device__ __forceinline__ float load(const T *p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(T *p, float v) { *p = __float2bfloat16_rn(v); }
};

template <int DT>
__global__ void __launch_bounds__(256) gemm_simt_kernel(int M, int N, int K, const typename Elem<DT>::T *__restrict__ A,
                                                        long long lda, long long strideA,
                                                        const typename Elem<DT>::T *__restrict__ B, long long ldb,
                                                        long long strideB, typename Elem<DT>::T *__restrict__ C,
                                                        long long ldc, long long strideC,
                                                        const typename Elem<DT>::T *__restrict__ bias, int act, long long a_cs,
                                                        long long b_cs)
{
    constexpr int TM = 64, TN = 64, TK = 16;
    __shared__ float As[TK][TM + 1];
    __shared__ float Bs[TK][TN + 1];
    const int b = blockIdx.z;
    A += (long long)b * strideA;
    B += (long long)b * strideB;
    C += (long long)b * strideC;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += TK) {
        for (int i = threadIdx.x; i < TM * TK; i += 256) {
            const int r = i / TK, c = i % TK;
            const int gm = m0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? Elem<DT>::load(A + (long long)gm * lda + (long long)gk * a_cs) : 0.0f;
        }
        for (int i = threadIdx.x; i < TK * TN; i += 256) {
            const int r = i / TN, c = i % TN;
            const int gk = k0 + r, gn = n0 + c;
            Bs[r][c] = (gk < K && gn < N) ? Elem<DT>::load(B + (long long)gk * ldb + (long long)gn * b_cs) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], bb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bb[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) {
                float v = acc[i][j];
                if (bias) v += Elem<DT>::load(bias + gn);
                if (act == 1) v = fmaxf(v, 0.0f);
                Elem<DT>::store(C + (long long)gm * ldc + gn, v);
            }
        }
    }
}

int launch_gemm_simt(int dtype, cudaStream_t st, int batch, int M, int N, int K, const void *A, long long lda,
                     long long strideA, const void *B, long long ldb, long long strideB, void *C, long long ldc,
                     long long strideC, const void *bias, int act, long long a_cs, long long b_cs)
{
    if (M == 0 || N == 0 || batch == 0) return BTM_OK;
    const long long gy = (M + 63) / 64, gx = (N + 63) / 64;
    if (gy > 65535 || batch > 65535) return set_error(BTM_ERR_UNSUPPORTED, "general kernel: M or batch too large for its grid");
    dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)batch);
    switch (dtype) {
    case BTM_F32:
        gemm_simt_kernel<BTM_F32><<<grid, 256, 0, st>>>(M, N, K, (const float *)A, lda, strideA, (const float *)B, ldb, strideB,
                                                        (float *)C, ldc, strideC, (const float *)bias, act, a_cs, b_cs);
        break;
    case BTM_F16:
        gemm_simt_kernel<BTM_F16><<<grid, 256, 0, st>>>(M, N, K, (const __half *)A, lda, strideA, (const __half *)B, ldb, strideB,
                                                        (__half *)C, ldc, strideC, (const __half *)bias, act, a_cs, b_cs);
        break;
    case BTM_BF16:
        gemm_simt_kernel<BTM_BF16><<<grid, 256, 0, st>>>(M, N, K, (const __nv_bfloat16 *)A, lda, strideA, (const __nv_bfloat16 *)B,
                                                         ldb, strideB, (__nv_bfloat16 *)C, ldc, strideC, (const __nv_bfloat16 *)bias, act, a_cs, b_cs);
        break;
    default:
        return set_error(BTM_ERR_UNSUPPORTED, "matmul: dtype %d is not supported", dtype);
    }
    return check_cuda(cudaGetLastError(), "gemm_simt launch");
}

} // namespace btm
