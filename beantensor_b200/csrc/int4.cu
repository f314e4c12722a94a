// int4 weight-only kernels.
//
// Storage (this build's addition to the reference dtype list, which has no sub-byte type):
// W[n,k] is a signed two's-complement nibble; byte n*(K/2) + k/2 holds even k in bits 0-3 and
// odd k in bits 4-7; one fp16 scale per `group` consecutive k, row-major [N, K/group].
//
// int4_gemv_kernel (M <= 8 per launch row-block) is a weight-streaming kernel: the packed
// weights are read exactly once with 128-bit loads, unpacked to exact fp16 integers in
// registers, and multiplied with the activations by mma.sync m16n8k16 (16 weight rows x 8
// activation rows per instruction, fp32 accumulation). Per 128-k block the fp32 partial sums
// are multiplied by the group scale and added to the running total, so the arithmetic is
//   out[m,n] = f16_rne( sum_g float(S[n,g]) * sum_{k in g} float(act[m,k]) * W[n,k] ).
// The sum over k inside an mma is order-free, which lets every lane keep the 32 consecutive
// nibbles of one 128-bit load: lane (g,t) of a warp owns weight rows g and g+8 and the k range
// [t*32, t*32+32) of each 128-k block; activations are staged in shared memory already permuted
// into the matching slot order.
#include <cuda_fp16.h>

#include "btm_internal.h"

namespace btm {

constexpr int GEMV_ROWS = 16;   // weight rows per CTA (= mma M)
constexpr int GEMV_WARPS = 4;   // 128-k blocks are dealt round-robin to the warps
constexpr int GEMV_UNROLL = 4;  // 128-k blocks in flight per warp

__device__ __forceinline__ uint4 ldg_stream(const uint4 *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Eight nibbles of one 32-bit word -> four half2 of exact signed values, as the pairs
// {k0,k4}, {k1,k5}, {k2,k6}, {k3,k7}. `x` must already be XORed with 0x88888888 so that each
// nibble holds value + 8. (1024 + n) - 1032 and (1024 + 16 n) / 16 - 72 are exact in fp16.
__device__ __forceinline__ void unpack8(uint32_t x, uint32_t (&h)[4])
{
    const uint32_t MAGIC = 0x64006400u; // half2(1024, 1024)
    const __half2 k1032 = __half2half2(__ushort_as_half((unsigned short)0x6408));
    const __half2 k16th = __half2half2(__ushort_as_half((unsigned short)0x2C00));  // 1/16
    const __half2 km72 = __half2half2(__ushort_as_half((unsigned short)0xD480));   // -72
    uint32_t lo0 = (x & 0x000F000Fu) | MAGIC;
    uint32_t hi0 = (x & 0x00F000F0u) | MAGIC;
    const uint32_t y = x >> 8;
    uint32_t lo1 = (y & 0x000F000Fu) | MAGIC;
    uint32_t hi1 = (y & 0x00F000F0u) | MAGIC;
    __half2 r0 = __hsub2(*reinterpret_cast<__half2 *>(&lo0), k1032);
    __half2 r1 = __hfma2(*reinterpret_cast<__half2 *>(&hi0), k16th, km72);
    __half2 r2 = __hsub2(*reinterpret_cast<__half2 *>(&lo1), k1032);
    __half2 r3 = __hfma2(*reinterpret_cast<__half2 *>(&hi1), k16th, km72);
    h[0] = *reinterpret_cast<uint32_t *>(&r0);
    h[1] = *reinterpret_cast<uint32_t *>(&r1);
    h[2] = *reinterpret_cast<uint32_t *>(&r2);
    h[3] = *reinterpret_cast<uint32_t *>(&r3);
}

__global__ void __launch_bounds__(GEMV_WARPS * 32)
int4_gemv_kernel(int M, int N, int K, int group, const __half *__restrict__ act, const uint8_t *__restrict__ w,
                 const __half *__restrict__ scales, __half *__restrict__ out)
{
    extern __shared__ uint4 act_s[]; // [mrows][K/8 + 1] permuted activations, then the reduction buffer
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.y * 8;
    const int mrows = min(8, M - m0);
    const int n0 = blockIdx.x * GEMV_ROWS;
    const int rowA = min(n0 + g, N - 1), rowB = min(n0 + g + 8, N - 1);
    const int nkb = K / 128;  // 128-k blocks per row
    const int G = K / group;  // scales per row
    const int units = K / 32; // 16-byte units per weight row
    const uint4 *wA = reinterpret_cast<const uint4 *>(w) + (size_t)rowA * units + t;
    const uint4 *wB = reinterpret_cast<const uint4 *>(w) + (size_t)rowB * units + t;
    const __half *sA = scales + (size_t)rowA * G;
    const __half *sB = scales + (size_t)rowB * G;

    uint4 qa[GEMV_UNROLL], qb[GEMV_UNROLL];
    float fa[GEMV_UNROLL], fb[GEMV_UNROLL];
    // First batch of weight loads goes out before the activations are staged.
#pragma unroll
    for (int u = 0; u < GEMV_UNROLL; ++u) {
        const int kb = warp + GEMV_WARPS * u;
        if (kb < nkb) {
            qa[u] = ldg_stream(wA + kb * 4);
            qb[u] = ldg_stream(wB + kb * 4);
            const int si = (kb * 128) / group;
            fa[u] = __half2float(__ldg(sA + si));
            fb[u] = __half2float(__ldg(sB + si));
        }
    }

    // Stage activations: 8 consecutive k -> [k0,k4,k1,k5,k2,k6,k3,k7], one padded row per m.
    const int row_u4 = K / 8 + 1;
    for (int i = threadIdx.x; i < mrows * (K / 8); i += blockDim.x) {
        const int m = i / (K / 8), j = i - m * (K / 8);
        const uint4 r = __ldg(reinterpret_cast<const uint4 *>(act + (size_t)(m0 + m) * K) + j);
        uint4 o;
        o.x = __byte_perm(r.x, r.z, 0x5410);
        o.y = __byte_perm(r.x, r.z, 0x7632);
        o.z = __byte_perm(r.y, r.w, 0x5410);
        o.w = __byte_perm(r.y, r.w, 0x7632);
        act_s[m * row_u4 + j] = o;
    }
    __syncthreads();

    float tot[4] = {0.f, 0.f, 0.f, 0.f};
    const bool has_b = g < mrows;
    const uint4 *arow = act_s + (has_b ? g : 0) * row_u4 + t * 4;

    for (int kb0 = warp; kb0 < nkb; kb0 += GEMV_WARPS * GEMV_UNROLL) {
        uint4 ca[GEMV_UNROLL], cb[GEMV_UNROLL];
        float sa[GEMV_UNROLL], sb[GEMV_UNROLL];
#pragma unroll
        for (int u = 0; u < GEMV_UNROLL; ++u) {
            ca[u] = qa[u];
            cb[u] = qb[u];
            sa[u] = fa[u];
            sb[u] = fb[u];
        }
        // Prefetch the next batch while this one is consumed.
#pragma unroll
        for (int u = 0; u < GEMV_UNROLL; ++u) {
            const int kb = kb0 + GEMV_WARPS * (GEMV_UNROLL + u);
            if (kb < nkb) {
                qa[u] = ldg_stream(wA + kb * 4);
                qb[u] = ldg_stream(wB + kb * 4);
                const int si = (kb * 128) / group;
                fa[u] = __half2float(__ldg(sA + si));
                fb[u] = __half2float(__ldg(sB + si));
            }
        }
#pragma unroll
        for (int u = 0; u < GEMV_UNROLL; ++u) {
            const int kb = kb0 + GEMV_WARPS * u;
            if (kb >= nkb) break;
            float c[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t xa[4] = {ca[u].x, ca[u].y, ca[u].z, ca[u].w};
            const uint32_t xb[4] = {cb[u].x, cb[u].y, cb[u].z, cb[u].w};
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
                uint32_t ha[4], hb[4];
                unpack8(xa[wd] ^ 0x88888888u, ha);
                unpack8(xb[wd] ^ 0x88888888u, hb);
                uint4 bv = make_uint4(0u, 0u, 0u, 0u);
                if (has_b) bv = arow[kb * 16 + wd];
                mma_16816(c, ha[0], hb[0], ha[1], hb[1], bv.x, bv.y);
                mma_16816(c, ha[2], hb[2], ha[3], hb[3], bv.z, bv.w);
            }
            tot[0] = fmaf(sa[u], c[0], tot[0]);
            tot[1] = fmaf(sa[u], c[1], tot[1]);
            tot[2] = fmaf(sb[u], c[2], tot[2]);
            tot[3] = fmaf(sb[u], c[3], tot[3]);
        }
    }

    // Cross-warp reduction through shared memory (reuses the activation buffer).
    __syncthreads();
    float *red = reinterpret_cast<float *>(act_s); // [warp][16 rows][8 m]
    red[(warp * 16 + g) * 8 + 2 * t] = tot[0];
    red[(warp * 16 + g) * 8 + 2 * t + 1] = tot[1];
    red[(warp * 16 + g + 8) * 8 + 2 * t] = tot[2];
    red[(warp * 16 + g + 8) * 8 + 2 * t + 1] = tot[3];
    __syncthreads();
    {
        const int m = threadIdx.x >> 4, r = threadIdx.x & 15; // 8 m x 16 rows = 128 threads
        float s = 0.f;
#pragma unroll
        for (int wi = 0; wi < GEMV_WARPS; ++wi) s += red[(wi * 16 + r) * 8 + m];
        if (m < mrows && n0 + r < N) out[(size_t)(m0 + m) * N + n0 + r] = __float2half_rn(s);
    }
}

// Any K (even), any group that divides K, any alignment: one thread per output, same arithmetic.
__global__ void int4_matmul_general_kernel(int M, int N, int K, int group, const __half *__restrict__ act,
                                           const uint8_t *__restrict__ w, const __half *__restrict__ scales,
                                           __half *__restrict__ out)
{
    const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (idx >= (long long)M * N) return;
    const int m = (int)(idx / N), n = (int)(idx - (long long)m * N);
    const int G = K / group;
    float total = 0.f;
    for (int gi = 0; gi < G; ++gi) {
        float part = 0.f;
        for (int k = gi * group; k < (gi + 1) * group; ++k) {
            const uint8_t b = w[(size_t)n * (K / 2) + k / 2];
            const int v = (k & 1) ? (int)((b >> 4) ^ 8) - 8 : (int)((b & 0xF) ^ 8) - 8;
            part = fmaf(__half2float(act[(size_t)m * K + k]), (float)v, part);
        }
        total = fmaf(__half2float(scales[(size_t)n * G + gi]), part, total);
    }
    out[idx] = __float2half_rn(total);
}

__global__ void int4_dequant_kernel(long long nbytes, int K, int group, const uint8_t *__restrict__ w,
                                    const __half *__restrict__ scales, __half *__restrict__ out)
{
    // One thread per packed 32-bit word (8 weights) -> one 16-byte store.
    const long long words = nbytes / 4;
    const int G = K / group;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < words; i += (long long)gridDim.x * blockDim.x) {
        const uint32_t x = __ldg(reinterpret_cast<const uint32_t *>(w) + i);
        const long long e0 = i * 8; // first element index
        const long long n = e0 / K;
        const int k0 = (int)(e0 - n * K);
        const float s = __half2float(__ldg(scales + n * G + k0 / group)); // 8 | group: one scale per word
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int lo = (int)(((x >> (8 * j)) & 0xF) ^ 8) - 8;
            const int hi = (int)(((x >> (8 * j + 4)) & 0xF) ^ 8) - 8;
            __half2 h = __floats2half2_rn((float)lo * s, (float)hi * s);
            o[j] = *reinterpret_cast<uint32_t *>(&h);
        }
        reinterpret_cast<uint4 *>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

__global__ void int4_dequant_general_kernel(long long numel, int K, int group, const uint8_t *__restrict__ w,
                                            const __half *__restrict__ scales, __half *__restrict__ out)
{
    const int G = K / group;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < numel; e += (long long)gridDim.x * blockDim.x) {
        const long long n = e / K;
        const int k = (int)(e - n * K);
        const uint8_t b = w[n * (K / 2) + k / 2];
        const int v = (k & 1) ? (int)((b >> 4) ^ 8) - 8 : (int)((b & 0xF) ^ 8) - 8;
        out[e] = __float2half_rn((float)v * __half2float(scales[n * G + k / group]));
    }
}

__global__ void int4_unpack_kernel(long long nbytes, const uint8_t *__restrict__ w, int8_t *__restrict__ out)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nbytes; i += (long long)gridDim.x * blockDim.x) {
        const uint8_t b = w[i];
        char2 v;
        v.x = (signed char)((int)((b & 0xF) ^ 8) - 8);
        v.y = (signed char)((int)((b >> 4) ^ 8) - 8);
        reinterpret_cast<char2 *>(out)[i] = v;
    }
}

static int grid_for(long long items, int block, int sm_cap)
{
    long long g = (items + block - 1) / block;
    if (g > sm_cap) g = sm_cap;
    if (g < 1) g = 1;
    return (int)g;
}

int launch_int4_gemv(cudaStream_t st, int sm_count, int M, int N, int K, int group, const void *act, const void *w,
                     const void *scales, void *out)
{
    (void)sm_count;
    if (M == 0 || N == 0) return BTM_OK;
    const bool fast = (K % 128 == 0) && (group % 128 == 0) && (((uintptr_t)act & 15) == 0) && (((uintptr_t)w & 15) == 0) &&
                      (((uintptr_t)scales & 1) == 0) && K > 0;
    if (!fast) {
        const long long total = (long long)M * N;
        const int block = 128;
        const long long grid = (total + block - 1) / block;
        if (grid > 0x7FFFFFFFLL) return set_error(BTM_ERR_UNSUPPORTED, "int4 matmul: output too large");
        int4_matmul_general_kernel<<<(unsigned)grid, block, 0, st>>>(M, N, K, group, (const __half *)act, (const uint8_t *)w,
                                                                     (const __half *)scales, (__half *)out);
        return check_cuda(cudaGetLastError(), "int4 general launch");
    }
    const int mrows = M < 8 ? M : 8;
    size_t smem = (size_t)mrows * (K / 8 + 1) * sizeof(uint4);
    const size_t red = GEMV_WARPS * 16 * 8 * sizeof(float);
    if (smem < red) smem = red;
    if (smem > 200 * 1024) return set_error(BTM_ERR_UNSUPPORTED, "int4 matmul: K=%d too large for the activation stage", K);
    if (smem > 48 * 1024) {
        int rc = check_cuda(cudaFuncSetAttribute(int4_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024),
                            "cudaFuncSetAttribute(int4_gemv)");
        if (rc) return rc;
    }
    dim3 grid((unsigned)((N + GEMV_ROWS - 1) / GEMV_ROWS), (unsigned)((M + 7) / 8));
    int4_gemv_kernel<<<grid, GEMV_WARPS * 32, smem, st>>>(M, N, K, group, (const __half *)act, (const uint8_t *)w,
                                                          (const __half *)scales, (__half *)out);
    return check_cuda(cudaGetLastError(), "int4 gemv launch");
}

int launch_int4_dequant(cudaStream_t st, int N, int K, int group, const void *w, const void *scales, void *out)
{
    const long long numel = (long long)N * K;
    if (numel == 0) return BTM_OK;
    const bool fast = (K % 8 == 0) && (group % 8 == 0) && (((uintptr_t)w & 3) == 0) && (((uintptr_t)out & 15) == 0);
    if (fast) {
        const long long nbytes = numel / 2;
        int4_dequant_kernel<<<grid_for(nbytes / 4, 256, 148 * 16), 256, 0, st>>>(nbytes, K, group, (const uint8_t *)w,
                                                                                (const __half *)scales, (__half *)out);
    } else {
        int4_dequant_general_kernel<<<grid_for(numel, 256, 148 * 16), 256, 0, st>>>(numel, K, group, (const uint8_t *)w,
                                                                                  (const __half *)scales, (__half *)out);
    }
    return check_cuda(cudaGetLastError(), "int4 dequant launch");
}

int launch_int4_unpack(cudaStream_t st, int N, int K, const void *w, void *out)
{
    const long long nbytes = (long long)N * K / 2;
    if (nbytes == 0) return BTM_OK;
    if (((uintptr_t)out & 1) != 0) return set_error(BTM_ERR_INVALID, "int4 unpack: output must be 2-byte aligned");
    int4_unpack_kernel<<<grid_for(nbytes, 256, 148 * 16), 256, 0, st>>>(nbytes, (const uint8_t *)w, (int8_t *)out);
    return check_cuda(cudaGetLastError(), "int4 unpack launch");
}

} // namespace btm
