// int4 weight-only GEMV for M <= 8, register-resident form.
//
// The kernel is a weight stream: N*K/2 bytes are read once and every byte is used once, so its time is the
// number of bytes it can keep in flight from HBM, and everything else has to stay out of the way of that.
//   * A warp owns 16 whole weight rows (one m16n8k16 mma's A rows) over a contiguous K slice of at most NB
//     128-k blocks. Lane (g, t) owns rows g and g + 8 and, of every 128-k block, the 32 consecutive nibbles
//     [32 t, 32 t + 32): one 128-bit global load per row and block. ALL of a warp's loads are issued before
//     anything else happens (2 x NB loads of 16 bytes per lane, straight into registers, no shared-memory
//     ring, no mbarrier): with ten warps per SM that is 160 KB per SM requested from HBM in the first few
//     hundred cycles.
//   * While those loads fly, the CTA stages the activations once: 8 consecutive values a0..a7 become the
//     pairs {a0,a4} {a1,a5}/16 {a2,a6} {a3,a7}/16, the slot order in which the nibbles of a 32-bit word
//     fall out of two masks and a shift (the k order inside an mma is free as long as both operands agree).
//   * The nibbles are NOT converted to their signed values. (x & 0x000F000F) ^ 0x64086408 is the fp16 pair
//     {1032 + v, 1032 + v'} and (x & 0x00F000F0) ^ 0x64806480 is {1152 + 16 v, 1152 + 16 v'}; multiplied with
//     a and a/16 both give a*v plus a constant that depends on the activations only:
//         corr[m, block] = 1032 * sum(a over even k) + 1152 * sum(a/16 over odd k).
//     corr is computed once per CTA while staging and enters the mma as the negated initial accumulator, so
//     the accumulator ends at sum(a*v) and the inner loop holds five logic instructions per eight weights and
//     one mma per 256, nothing else. The accumulator passes through values near 5e4 on the way, which costs
//     about 1e-4 relative accuracy in fp32 (measured; the bound of the path is 2e-3).
//   * Per 128-k block the partial sum is scaled by the two rows' group scales (fp32) and added to the running
//     total. The warps that share a row group (K longer than NB blocks) meet once per row group in shared
//     memory (a named barrier among those warps only) and their first warp rounds and stores.
// Programmatic dependent launch: weights and scales are requested before griddepcontrol.wait (they are
// parameters that no predecessor of this kind writes), activations and output are touched after it.
#include <cuda_fp16.h>

#include <cstring>

#include "btm_internal.h"

namespace btm {

namespace {

constexpr int GR_ROWS = 16; // weight rows per warp = rows of the mma's A operand

template <int NB>
struct RowsCfg {
    static constexpr int kWarps = NB == 16 ? 10 : 20; // 2 * NB * 4 registers of weights per lane: 128 or 64
    static constexpr int kThreads = kWarps * 32;
};

__device__ __forceinline__ uint4 ldg_stream(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lop_and_xor(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); // (a & b) ^ c
    return r;
}
__device__ __forceinline__ void mma_acc(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
__device__ __forceinline__ float f16_lo(uint32_t v) { return __half2float(__ushort_as_half((unsigned short)(v & 0xFFFFu))); }
__device__ __forceinline__ float f16_hi(uint32_t v) { return __half2float(__ushort_as_half((unsigned short)(v >> 16))); }

// kVecScale: a warp's scales (NB consecutive fp16 per row) are fetched with 128-bit loads up front; otherwise one
// 16-bit load per row and block inside the loop (any group size that is a multiple of 128, any K slice).
template <int NB, bool kVecScale>
__global__ void __launch_bounds__(RowsCfg<NB>::kThreads, 1)
int4_gemv_rows_kernel(const uint8_t *__restrict__ w, int M, int N, int K, int bpg, const __half *__restrict__ act,
                      const __half *__restrict__ scales, __half *__restrict__ out, int ksplit, int teams)
{
    constexpr int kWarps = RowsCfg<NB>::kWarps;
    // Shared memory: [M][K/8 + 4] uint4 staged activations | [K/128][8] fp32 corrections | [warps][16 rows][8 m] fp32 partials
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int nkb = K >> 7;
    const int G = nkb / bpg; // scales per row
    const int pitch = (K >> 3) + 4; // uint4 per staged activation row: 64 bytes mod 128, so that two rows fill one access phase
    uint4 *act_s = reinterpret_cast<uint4 *>(smem);
    float *corr_s = reinterpret_cast<float *>(smem + (size_t)M * pitch * 16);
    float *red_s = corr_s + nkb * 8;
    const int team = warp / ksplit, kslot = warp - team * ksplit;
    const int nbw = (nkb + ksplit - 1) / ksplit;          // 128-k blocks per warp (<= NB)
    const int kb0 = kslot * nbw;
    const int nb = team < teams ? max(0, min(nbw, nkb - kb0)) : 0;
    const int nrg = (N + GR_ROWS - 1) / GR_ROWS;
    const int rg_stride = teams * (int)gridDim.x;
    int rg = team * (int)gridDim.x + (int)blockIdx.x;
    const size_t row_bytes = (size_t)(K >> 1);

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    uint4 qa[NB], qb[NB];
    uint32_t sva[NB / 2], svb[NB / 2]; // kVecScale: the warp's NB scales per row, two fp16 per word
    // Scales of blocks 8 j8 .. 8 j8 + 7 of both rows. The first eight are requested with the weights; the second eight
    // (NB = 16) after the first blocks have been consumed and their registers are free again.
    auto load_scales = [&](int rgi, int j8) {
        if (j8 * 8 < nb) {
            const int ra = min(rgi * GR_ROWS + g, N - 1), rb = min(rgi * GR_ROWS + g + 8, N - 1);
            const uint4 a = ldg_stream(scales + (size_t)ra * G + kb0 + j8 * 8), b = ldg_stream(scales + (size_t)rb * G + kb0 + j8 * 8);
            sva[4 * j8] = a.x, sva[4 * j8 + 1] = a.y, sva[4 * j8 + 2] = a.z, sva[4 * j8 + 3] = a.w;
            svb[4 * j8] = b.x, svb[4 * j8 + 1] = b.y, svb[4 * j8 + 2] = b.z, svb[4 * j8 + 3] = b.w;
        }
    };
    auto issue_loads = [&](int rgi) {
        const int ra = min(rgi * GR_ROWS + g, N - 1), rb = min(rgi * GR_ROWS + g + 8, N - 1); // rows past N are clamped, never stored
        const uint8_t *pa = w + (size_t)ra * row_bytes + (size_t)kb0 * 64 + t * 16;
        const uint8_t *pb = w + (size_t)rb * row_bytes + (size_t)kb0 * 64 + t * 16;
#pragma unroll
        for (int j = 0; j < NB; ++j)
            if (j < nb) {
                qa[j] = ldg_stream(pa + j * 64);
                qb[j] = ldg_stream(pb + j * 64);
            }
        if constexpr (kVecScale) load_scales(rgi, 0);
    };
    bool have = team < teams && rg < nrg; // every warp of a team takes the same path (a warp without blocks contributes zeros)
    if (have) issue_loads(rg);

    // ---------------------------------------------------------------- activations (after the predecessor has finished)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    {
        const int per_row = K >> 3; // uint4 (8 activations) per row
        const int total = M * per_row;
        for (int i = threadIdx.x; i < nkb * 8; i += kWarps * 32)
            if ((i & 7) >= M) corr_s[i] = 0.0f;
        const __half2 sixteenth = __half2half2(__ushort_as_half((unsigned short)0x2C00));
        for (int base = warp * 32; base < total; base += kWarps * 32) {
            const int i = base + lane;
            const bool valid = i < total;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (valid) v = __ldg(reinterpret_cast<const uint4 *>(act) + i);
            const int m = i / per_row, r = i - m * per_row;
            const int kb = r >> 4, tt = (r >> 2) & 3, wd = r & 3;
            uint4 o;
            o.x = __byte_perm(v.x, v.z, 0x5410);
            uint32_t b15 = __byte_perm(v.x, v.z, 0x7632);
            o.z = __byte_perm(v.y, v.w, 0x5410);
            uint32_t b37 = __byte_perm(v.y, v.w, 0x7632);
            __half2 h15 = __hmul2(*reinterpret_cast<__half2 *>(&b15), sixteenth);
            __half2 h37 = __hmul2(*reinterpret_cast<__half2 *>(&b37), sixteenth);
            o.y = *reinterpret_cast<uint32_t *>(&h15);
            o.w = *reinterpret_cast<uint32_t *>(&h37);
            if (valid) act_s[(size_t)m * pitch + kb * 16 + wd * 4 + tt] = o;
            float part = 1032.0f * ((f16_lo(o.x) + f16_hi(o.x)) + (f16_lo(o.z) + f16_hi(o.z))) +
                         1152.0f * ((f16_lo(o.y) + f16_hi(o.y)) + (f16_lo(o.w) + f16_hi(o.w)));
            // the 16 lanes of a half-warp hold the 16 words of one (row, block)
            part += __shfl_xor_sync(0xffffffffu, part, 8);
            part += __shfl_xor_sync(0xffffffffu, part, 4);
            part += __shfl_xor_sync(0xffffffffu, part, 2);
            part += __shfl_xor_sync(0xffffffffu, part, 1);
            if (valid && (lane & 15) == 0) corr_s[kb * 8 + m] = part;
        }
    }
    __syncthreads();

    const bool has_row = g < M; // lane (g, t) supplies activation row g to the mma's B operand
    const uint32_t act_u32 = (uint32_t)__cvta_generic_to_shared(act_s) + (uint32_t)((min(g, M - 1) * pitch + t) * 16);
    const float *corr_t = corr_s + 2 * t;
    float *red_mine = red_s + warp * 128;

    while (have) {
        float tot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            if constexpr (kVecScale && NB > 8) {
                if (j == 2) load_scales(rg, 1);
            }
            if (j < nb) {
                const int kb = kb0 + j;
                const uint32_t xa[4] = {qa[j].x, qa[j].y, qa[j].z, qa[j].w};
                const uint32_t xb[4] = {qb[j].x, qb[j].y, qb[j].z, qb[j].w};
                const float2 cr = *reinterpret_cast<const float2 *>(corr_t + kb * 8);
                float c0[4] = {-cr.x, -cr.y, -cr.x, -cr.y}, c1[4];
#pragma unroll
                for (int wd = 0; wd < 4; ++wd) {
                    uint4 av = make_uint4(0u, 0u, 0u, 0u);
                    if (has_row) av = lds_v4(act_u32 + (uint32_t)((kb * 16 + wd * 4) * 16));
                    const uint32_t ya = xa[wd] >> 8, yb = xb[wd] >> 8;
                    const uint32_t la0 = lop_and_xor(xa[wd], 0x000F000Fu, 0x64086408u), ha0 = lop_and_xor(xa[wd], 0x00F000F0u, 0x64806480u);
                    const uint32_t lb0 = lop_and_xor(xb[wd], 0x000F000Fu, 0x64086408u), hb0 = lop_and_xor(xb[wd], 0x00F000F0u, 0x64806480u);
                    const uint32_t la1 = lop_and_xor(ya, 0x000F000Fu, 0x64086408u), ha1 = lop_and_xor(ya, 0x00F000F0u, 0x64806480u);
                    const uint32_t lb1 = lop_and_xor(yb, 0x000F000Fu, 0x64086408u), hb1 = lop_and_xor(yb, 0x00F000F0u, 0x64806480u);
                    mma_acc(c0, la0, lb0, ha0, hb0, av.x, av.y);
                    if (wd == 0) mma_zero(c1, la1, lb1, ha1, hb1, av.z, av.w);
                    else mma_acc(c1, la1, lb1, ha1, hb1, av.z, av.w);
                }
                float sa, sb;
                if constexpr (kVecScale) {
                    const uint32_t wa = sva[j >> 1], wb = svb[j >> 1];
                    sa = (j & 1) ? f16_hi(wa) : f16_lo(wa);
                    sb = (j & 1) ? f16_hi(wb) : f16_lo(wb);
                } else {
                    const int ra = min(rg * GR_ROWS + g, N - 1), rb = min(rg * GR_ROWS + g + 8, N - 1);
                    const int si = bpg == 1 ? kb : kb / bpg;
                    sa = __half2float(__ldg(scales + (size_t)ra * G + si));
                    sb = __half2float(__ldg(scales + (size_t)rb * G + si));
                }
                tot[0] = fmaf(sa, c0[0] + c1[0], tot[0]);
                tot[1] = fmaf(sa, c0[1] + c1[1], tot[1]);
                tot[2] = fmaf(sb, c0[2] + c1[2], tot[2]);
                tot[3] = fmaf(sb, c0[3] + c1[3], tot[3]);
            }
        }
        // partials [row][m]: accumulator columns are m = 2t, 2t + 1
        *reinterpret_cast<float2 *>(red_mine + g * 8 + 2 * t) = make_float2(tot[0], tot[1]);
        *reinterpret_cast<float2 *>(red_mine + (g + 8) * 8 + 2 * t) = make_float2(tot[2], tot[3]);
        if (ksplit > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(ksplit * 32) : "memory");
        else __syncwarp();
        if (kslot == 0) {
            const int n0 = rg * GR_ROWS;
            const float *red_team = red_s + team * ksplit * 128;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int o = lane + 32 * i;
                const int m = o >> 4, r = o & 15;
                float sum = 0.f;
                for (int ks = 0; ks < ksplit; ++ks) sum += red_team[ks * 128 + r * 8 + m]; // fixed order: the result does not depend on timing
                if (m < M && n0 + r < N) out[(size_t)m * N + n0 + r] = __float2half_rn(sum);
            }
        }
        rg += rg_stride;
        have = rg < nrg;
        if (have) {
            issue_loads(rg);
            // the partials are rewritten next round: everyone must have read them
            if (ksplit > 1) asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(ksplit * 32) : "memory");
            else __syncwarp();
        }
    }
}

template <int NB>
size_t rows_smem_bytes(int M, int K)
{
    return (size_t)M * ((K >> 3) + 4) * 16 + (size_t)(K >> 7) * 8 * 4 + (size_t)RowsCfg<NB>::kWarps * 128 * 4;
}

template <int NB>
int launch_rows(cudaStream_t st, int sm_count, int M, int N, int K, int group, const void *act, const void *w, const void *scales,
                void *out)
{
    constexpr int kWarps = RowsCfg<NB>::kWarps;
    const int nkb = K / 128, bpg = group / 128, G = K / group;
    const int ksplit = (nkb + NB - 1) / NB;
    if (ksplit > kWarps) return -1;
    const int teams = kWarps / ksplit;
    const int nbw = (nkb + ksplit - 1) / ksplit;
    const size_t smem = rows_smem_bytes<NB>(M, K);
    if (smem > 200 * 1024) return -1;
    const bool vec = bpg == 1 && (G % 8) == 0 && (nkb % 8) == 0 && (nbw % 8) == 0 && (((uintptr_t)scales & 15) == 0);
    const int nrg = (N + GR_ROWS - 1) / GR_ROWS;
    const int want = (nrg + teams - 1) / teams;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(want < sm_count ? want : sm_count));
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization; // the kernel orders itself with griddepcontrol
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const uint8_t *w_b = (const uint8_t *)w;
    const __half *act_h = (const __half *)act, *sc_h = (const __half *)scales;
    __half *out_h = (__half *)out;
    int bpg_v = bpg, ksplit_v = ksplit, teams_v = teams;
    void *args[] = {(void *)&w_b, (void *)&M, (void *)&N, (void *)&K, (void *)&bpg_v, (void *)&act_h, (void *)&sc_h, (void *)&out_h,
                    (void *)&ksplit_v, (void *)&teams_v};
    const void *fn = vec ? (const void *)int4_gemv_rows_kernel<NB, true> : (const void *)int4_gemv_rows_kernel<NB, false>;
    cudaError_t e = cudaLaunchKernelExC(&cfg, fn, args);
    if (e != cudaSuccess) return check_cuda(e, "int4 gemv (rows) launch");
    return check_cuda(cudaGetLastError(), "int4 gemv (rows) launch");
}

} // namespace

int configure_int4_gemv_rows_kernels()
{
    cudaError_t e = cudaSuccess;
    const int lim = 200 * 1024;
    if (e == cudaSuccess) e = cudaFuncSetAttribute(int4_gemv_rows_kernel<16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(int4_gemv_rows_kernel<16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(int4_gemv_rows_kernel<8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(int4_gemv_rows_kernel<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    return check_cuda(e, "cudaFuncSetAttribute(int4_gemv_rows)");
}

// Returns a btm_status, or -1 when the shape is outside what this kernel takes (nothing launched, no error set):
// M in 1..8, K a multiple of 128, group a multiple of 128, 16-byte aligned weights and activations.
int launch_int4_gemv_rows(cudaStream_t st, int sm_count, int M, int N, int K, int group, const void *act, const void *w,
                          const void *scales, void *out, int nb)
{
    if (M < 1 || M > 8 || N < 1 || K < 128 || (K % 128) || group < 128 || (group % 128) || (K % group)) return -1;
    if ((((uintptr_t)act | (uintptr_t)w) & 15) || (((uintptr_t)scales | (uintptr_t)out) & 1)) return -1;
    if (nb == 8) return launch_rows<8>(st, sm_count, M, N, K, group, act, w, scales, out);
    return launch_rows<16>(st, sm_count, M, N, K, group, act, w, scales, out);
}

} // namespace btm
