// int4 weight-only GEMV for M <= 8 activation rows, register-resident form.
//
// The kernel is a weight stream: N*K/2 bytes are read once and every byte is used once. What it has to get right
// is (a) how many bytes it keeps in flight from HBM and (b) how few instructions it spends per byte, because on
// this part the arithmetic is not free: a mma.sync m16n8k16 issues once per 8 cycles per SM sub-partition and a
// logic instruction once per 2 (both measured), so the 45 M weights of the 11008 x 4096 workload cost at least
// 1.3 us of tensor issue and 1.6 us of logic issue per launch before anything else.
//   * Two persistent CTAs per SM, eight warps each. A CTA walks the 16-row weight groups c, c + grid, ...; its eight
//     warps split K (four 128-k blocks each at K = 4096). Lane (g, t) of a warp owns rows g and g + 8 and, of every
//     128-k block, the 32 consecutive nibbles [32 t, 32 t + 32): one 128-bit global load per row and block, straight
//     into registers. There is no shared-memory ring and no mbarrier. Every warp holds TWO register buffers: the
//     loads of the group after next are issued as soon as a buffer has been consumed, so two groups per CTA
//     (128 KB per SM) are in flight while a third is being multiplied.
//   * The activations are staged once per CTA (every warp the K slice it will use itself, so no CTA barrier precedes
//     the first product), permuted to the slot order in which the nibbles of a 32-bit word
//     fall out of two masks and a shift: 8 consecutive values a0..a7 become {a0,a4} {a1,a5}/16 {a2,a6} {a3,a7}/16
//     (the k order inside an mma is free as long as both operands agree).
//   * The nibbles are NOT converted to their signed values. (x & 0x000F000F) ^ 0x64086408 is the fp16 pair
//     {1032 + v, 1032 + v'} and (x & 0x00F000F0) ^ 0x64806480 is {1152 + 16 v, 1152 + 16 v'}; multiplied with a and
//     a/16 both give a*v plus a term that depends on the activations only:
//         corr[m, block] = 1032 * sum(a over even k) + 1152 * sum(a/16 over odd k),
//     computed while staging and handed to the mma as its (negated) initial accumulator. The inner loop is then five
//     logic instructions per eight weights, one mma per 256 and one shared-memory load per mma. The accumulator
//     passes through values near 5e4 on the way; the measured cost is 2.1e-4 relative error against the fp64 checker,
//     the same as the kernels that remove the offsets (the bound of the path is 2e-3).
//   * The four blocks of a warp run as four independent accumulator chains, interleaved, so that a mma never waits
//     for its predecessor (latency 20 cycles). Per block the sum is scaled by the two rows' group scales in fp32;
//     the eight warps of a CTA meet once per row group in shared memory and one of them rounds and stores.
// Programmatic dependent launch: weights and scales are requested before griddepcontrol.wait (they are parameters
// that no predecessor of this kind writes), activations and output are touched after it.
#include <cuda_fp16.h>

#include <cstring>

#include "btm_internal.h"

namespace btm {

namespace {

constexpr int GR_W = 8;   // warps per CTA = ways K is split
constexpr int GR_NB = 4;  // 128-k blocks per warp
constexpr int GR_THREADS = GR_W * 32;

__device__ __forceinline__ uint4 ldg_stream(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream2(const void *p)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
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
__device__ __forceinline__ float f16_lo(uint32_t v) { return __half2float(__ushort_as_half((unsigned short)(v & 0xFFFFu))); }
__device__ __forceinline__ float f16_hi(uint32_t v) { return __half2float(__ushort_as_half((unsigned short)(v >> 16))); }

__global__ void __launch_bounds__(GR_THREADS, 2)
int4_gemv_regs_kernel(const uint8_t *__restrict__ w, int M, int N, int K, const __half *__restrict__ act,
                      const __half *__restrict__ scales, __half *__restrict__ out)
{
    constexpr int NB = GR_NB, W = GR_W;
    // Shared memory: [M][K/8 + 4] uint4 staged activations | [K/128][4] float4 negated corrections | 2 x [8 warps][16 rows][8 m] partials
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int nkb = K >> 7;   // 128-k blocks per row = scales per row (group 128); a multiple of NB
    const int pitch = (K >> 3) + 4; // uint4 per staged row: 64 bytes mod 128, so that two rows fill one access phase
    uint4 *act_s = reinterpret_cast<uint4 *>(smem);
    float4 *corr_s = reinterpret_cast<float4 *>(smem + (size_t)M * pitch * 16);
    float *red_s = reinterpret_cast<float *>(corr_s + nkb * 4);
    const int kb0 = warp * NB;
    const bool active = kb0 < nkb; // K shorter than 4096: the last warps have no blocks and contribute zeros
    const int nrg = (N + 15) >> 4;
    const size_t row_bytes = (size_t)(K >> 1);
    const int grid = (int)gridDim.x;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    uint32_t qa0[NB * 4], qb0[NB * 4], sv0[4], qa1[NB * 4], qb1[NB * 4], sv1[4];
    auto issue_loads = [&](int rgi, uint32_t (&qa)[NB * 4], uint32_t (&qb)[NB * 4], uint32_t (&sv)[4]) {
        if (!active) return;
        const int ra = min(rgi * 16 + g, N - 1), rb = min(rgi * 16 + g + 8, N - 1); // rows past N are clamped, never stored
        const uint8_t *pa = w + (size_t)ra * row_bytes + (size_t)kb0 * 64 + t * 16;
        const uint8_t *pb = w + (size_t)rb * row_bytes + (size_t)kb0 * 64 + t * 16;
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const uint4 va = ldg_stream(pa + j * 64), vb = ldg_stream(pb + j * 64);
            qa[4 * j] = va.x, qa[4 * j + 1] = va.y, qa[4 * j + 2] = va.z, qa[4 * j + 3] = va.w;
            qb[4 * j] = vb.x, qb[4 * j + 1] = vb.y, qb[4 * j + 2] = vb.z, qb[4 * j + 3] = vb.w;
        }
        const uint2 a = ldg_stream2(scales + (size_t)ra * nkb + kb0), b = ldg_stream2(scales + (size_t)rb * nkb + kb0);
        sv[0] = a.x, sv[1] = a.y, sv[2] = b.x, sv[3] = b.y;
    };
    int rgA = blockIdx.x, rgB = blockIdx.x + grid;
    if (rgA < nrg) issue_loads(rgA, qa0, qb0, sv0);
    if (rgB < nrg) issue_loads(rgB, qa1, qb1, sv1);

    // ---------------------------------------------------------------- activations (after the predecessor has finished)
    // Every warp stages the activations of its own K slice (its NB blocks of every row) and nothing else, so the warps
    // do not meet on a CTA barrier before their first product: one round trip to L2, a permute, and the warp goes on.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (active) {
        const int per_row = K >> 3;          // uint4 (8 activations) per row
        constexpr int PER_WARP = NB * 16;    // uint4 of one row that belong to this warp's blocks
        const __half2 sixteenth = __half2half2(__ushort_as_half((unsigned short)0x2C00));
        for (int i = lane; i < NB * 16; i += 32) // corrections of rows m >= M: never stored, but defined
            if ((((i >> 2) & 3) * 2 + (i & 1)) >= M) reinterpret_cast<float *>(corr_s + kb0 * 4)[i] = 0.0f;
        constexpr int UN = 4; // loads in flight per lane
        const int total = M * PER_WARP;
        for (int base0 = 0; base0 < total; base0 += 32 * UN) {
            uint4 vv[UN];
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const int i = base0 + u * 32 + lane;
                const int m = i / PER_WARP, r = i - m * PER_WARP;
                vv[u] = make_uint4(0u, 0u, 0u, 0u);
                if (i < total) vv[u] = __ldg(reinterpret_cast<const uint4 *>(act) + (size_t)m * per_row + kb0 * 16 + r);
            }
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const int i = base0 + u * 32 + lane;
                const bool valid = i < total;
                const int m = i / PER_WARP, r = i - m * PER_WARP;
                const int kb = kb0 + (r >> 4), tt = (r >> 2) & 3, wd = r & 3;
                const uint4 v = vv[u];
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
                // stored as the initial accumulator of lane t = m / 2: {-c(2t), -c(2t+1), -c(2t), -c(2t+1)}
                if (valid && (lane & 15) == 0) {
                    float *c = reinterpret_cast<float *>(corr_s + kb * 4 + (m >> 1));
                    c[m & 1] = -part;
                    c[2 + (m & 1)] = -part;
                }
            }
        }
    }
    __syncwarp();

    // Lane (g, t) supplies activation row g to the mma's B operand; output columns m >= M are never stored, so
    // those lanes simply read the last row again.
    const uint32_t act_u32 = (uint32_t)__cvta_generic_to_shared(act_s) + (uint32_t)((min(g, M - 1) * pitch + t) * 16);
    const uint32_t corr_u32 = (uint32_t)__cvta_generic_to_shared(corr_s) + (uint32_t)(t * 16);

    auto compute = [&](const uint32_t (&qa)[NB * 4], const uint32_t (&qb)[NB * 4], const uint32_t (&sv)[4], float *red) {
        float tot[4] = {0.f, 0.f, 0.f, 0.f};
        if (active) {
            float c[NB][4];
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                uint4 cr;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(cr.x), "=r"(cr.y), "=r"(cr.z), "=r"(cr.w) : "r"(corr_u32 + (uint32_t)((kb0 + b) * 64)));
                c[b][0] = __uint_as_float(cr.x), c[b][1] = __uint_as_float(cr.y), c[b][2] = __uint_as_float(cr.z), c[b][3] = __uint_as_float(cr.w);
            }
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
                    for (int b = 0; b < NB; ++b) { // the four blocks are independent chains: consecutive mma never depend on each other
                        uint32_t xa = qa[4 * b + wd], xb = qb[4 * b + wd];
                        if (hf) {
                            xa >>= 8;
                            xb >>= 8;
                        }
                        uint2 av;
                        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(av.x), "=r"(av.y) : "r"(act_u32 + (uint32_t)(((kb0 + b) * 16 + wd * 4) * 16 + hf * 8)));
                        const uint32_t la = lop_and_xor(xa, 0x000F000Fu, 0x64086408u), ha = lop_and_xor(xa, 0x00F000F0u, 0x64806480u);
                        const uint32_t lb = lop_and_xor(xb, 0x000F000Fu, 0x64086408u), hb = lop_and_xor(xb, 0x00F000F0u, 0x64806480u);
                        mma_acc(c[b], la, lb, ha, hb, av.x, av.y);
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                const uint32_t wa = sv[b >> 1], wb = sv[2 + (b >> 1)];
                const float sa = (b & 1) ? f16_hi(wa) : f16_lo(wa);
                const float sb = (b & 1) ? f16_hi(wb) : f16_lo(wb);
                tot[0] = fmaf(sa, c[b][0], tot[0]);
                tot[1] = fmaf(sa, c[b][1], tot[1]);
                tot[2] = fmaf(sb, c[b][2], tot[2]);
                tot[3] = fmaf(sb, c[b][3], tot[3]);
            }
        }
        // partials [row][m]: accumulator columns are m = 2t, 2t + 1
        *reinterpret_cast<float2 *>(red + warp * 128 + g * 8 + 2 * t) = make_float2(tot[0], tot[1]);
        *reinterpret_cast<float2 *>(red + warp * 128 + (g + 8) * 8 + 2 * t) = make_float2(tot[2], tot[3]);
    };
    auto reduce_store = [&](const float *red, int n0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int o = lane + 32 * i;
            const int m = o >> 4, r = o & 15;
            float sum = 0.f;
#pragma unroll
            for (int ks = 0; ks < W; ++ks) sum += red[ks * 128 + r * 8 + m]; // fixed order: the result does not depend on timing
            if (m < M && n0 + r < N) out[(size_t)m * N + n0 + r] = __float2half_rn(sum);
        }
    };
    // Two sets of partials, one per register buffer: a set is rewritten only after a later barrier has been passed by
    // the warp that read it, so one barrier per row group is enough.
    float *red0 = red_s, *red1 = red_s + W * 128;
    while (rgA < nrg) {
        compute(qa0, qb0, sv0, red0);
        const int nA = rgA * 16;
        rgA += 2 * grid;
        if (rgA < nrg) issue_loads(rgA, qa0, qb0, sv0);
        __syncthreads();
        if (warp == 0) reduce_store(red0, nA);
        if (rgB >= nrg) break;
        compute(qa1, qb1, sv1, red1);
        const int nB = rgB * 16;
        rgB += 2 * grid;
        if (rgB < nrg) issue_loads(rgB, qa1, qb1, sv1);
        __syncthreads();
        if (warp == 1) reduce_store(red1, nB);
    }
}

size_t regs_smem_bytes(int M, int K)
{
    return (size_t)M * ((K >> 3) + 4) * 16 + (size_t)(K >> 7) * 64 + (size_t)2 * GR_W * 128 * 4;
}

} // namespace

int configure_int4_gemv_regs_kernels()
{
    return check_cuda(cudaFuncSetAttribute(int4_gemv_regs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024),
                      "cudaFuncSetAttribute(int4_gemv_regs)");
}

// Returns a btm_status, or -1 when the shape is outside what this kernel takes (nothing launched, no error set):
// M in 1..8 with the staged activations within half an SM's shared memory, K a multiple of 512 up to 4096, group 128,
// 16-byte aligned weights and activations, 8-byte aligned scales.
int launch_int4_gemv_regs(cudaStream_t st, int sm_count, int M, int N, int K, int group, const void *act, const void *w,
                          const void *scales, void *out)
{
    if (M < 1 || M > 8 || N < 1 || group != 128 || K < 512 || (K % 512) || K > 128 * GR_W * GR_NB) return -1;
    if ((((uintptr_t)act | (uintptr_t)w) & 15) || ((uintptr_t)scales & 7) || ((uintptr_t)out & 1)) return -1;
    const size_t smem = regs_smem_bytes(M, K);
    if (smem > 100 * 1024) return -1;
    const int nrg = (N + 15) / 16;
    const int want = 2 * sm_count;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(nrg < want ? nrg : want));
    cfg.blockDim = dim3(GR_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization; // the kernel orders itself with griddepcontrol
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, int4_gemv_regs_kernel, (const uint8_t *)w, M, N, K, (const __half *)act, (const __half *)scales,
                                       (__half *)out);
    if (e != cudaSuccess) return check_cuda(e, "int4 gemv (registers) launch");
    return check_cuda(cudaGetLastError(), "int4 gemv (registers) launch");
}

} // namespace btm
