// int4 weight-only kernels.
//
// Storage (this build's addition to the reference dtype list, which has no sub-byte type):
// W[n,k] is a signed two's-complement nibble; byte n*(K/2) + k/2 holds even k in bits 0-3 and
// odd k in bits 4-7; one fp16 scale per `group` consecutive k, row-major [N, K/group].
//
// int4_gemv_kernel (M <= 8 per launch row-block) is a weight-streaming kernel: the packed
// weights are read from HBM exactly once (bulk async copies into shared memory, issued for the
// CTA's whole slab at once), then fetched with 128-bit shared loads, unpacked to exact fp16 integers
// in registers, and multiplied with the activations by mma.sync m16n8k16 (16 weight rows x 8
// activation rows per instruction, fp32 accumulation). Per 128-k block the fp32 partial sums
// are multiplied by the group scale and added to the running total, so the arithmetic is
//   out[m,n] = f16_rne( sum_g float(S[n,g]) * sum_{k in g} float(act[m,k]) * W[n,k] ).
// The sum over k inside an mma is order-free, which lets every lane keep the 32 consecutive
// nibbles of one 128-bit load: lane (g,t) of a warp owns weight rows g and g+8 and the k range
// [t*32, t*32+32) of each 128-k block; the matching activations are read from global memory (L1
// hits after the first touch) and permuted into the same slot order with two byte-permutes per pair.
#include <cuda_fp16.h>

#include "btm_internal.h"
#include "btm_ptx.cuh"
#include "int4_unpack.cuh"

namespace btm {

constexpr int GEMV_ROWS = 16;   // weight rows per CTA (= mma M)
constexpr int GEMV_WARPS = 4;   // 128-k blocks are dealt round-robin to the warps

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// (a & b) ^ c in one LOP3.
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); // 0x6a = (a & b) ^ c
    return r;
}

// First mma of a chain: accumulator input is zero.
__device__ __forceinline__ void mma_16816_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                                uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// Eight two's-complement nibbles of one 32-bit word -> four half2 of exact signed values, as the
// pairs {k0,k4}, {k1,k5}, {k2,k6}, {k3,k7}. (x & mask) ^ (0x64006400 | sign bits) builds the fp16
// numbers 1024 + (n ^ 8) = 1032 + value (low nibbles) or 1024 + 16 (n ^ 8) = 1152 + 16 value (high
// nibbles) in one LOP3 each; one HADD2 / HFMA2 per pair then removes the offset exactly.
__device__ __forceinline__ void unpack8(uint32_t x, uint32_t (&h)[4])
{
    const __half2 k1032 = __half2half2(__ushort_as_half((unsigned short)0x6408));
    const __half2 k16th = __half2half2(__ushort_as_half((unsigned short)0x2C00));  // 1/16
    const __half2 km72 = __half2half2(__ushort_as_half((unsigned short)0xD480));   // -72
    uint32_t lo0 = and_xor(x, 0x000F000Fu, 0x64086408u);
    uint32_t hi0 = and_xor(x, 0x00F000F0u, 0x64806480u);
    const uint32_t y = x >> 8;
    uint32_t lo1 = and_xor(y, 0x000F000Fu, 0x64086408u);
    uint32_t hi1 = and_xor(y, 0x00F000F0u, 0x64806480u);
    __half2 r0 = __hsub2(*reinterpret_cast<__half2 *>(&lo0), k1032);
    __half2 r1 = __hfma2(*reinterpret_cast<__half2 *>(&hi0), k16th, km72);
    __half2 r2 = __hsub2(*reinterpret_cast<__half2 *>(&lo1), k1032);
    __half2 r3 = __hfma2(*reinterpret_cast<__half2 *>(&hi1), k16th, km72);
    h[0] = *reinterpret_cast<uint32_t *>(&r0);
    h[1] = *reinterpret_cast<uint32_t *>(&r1);
    h[2] = *reinterpret_cast<uint32_t *>(&r2);
    h[3] = *reinterpret_cast<uint32_t *>(&r3);
}

// Bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned) global -> shared memory of this
// CTA, completion counted on `bar`.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

constexpr int GEMV_ROW_PAD = 64;      // int4_gemm_mma_kernel: bytes between staged rows beyond K/2
constexpr int GEMV_PIECE_BYTES = 16 * 128; // int4_gemv_kernel: one TMA piece = 16 rows x 256 k
constexpr int GEMV_MAX_PIECES = 64;   // K <= 16384 on the fast GEMV path

template <bool kStageAct>
__global__ void __launch_bounds__(GEMV_WARPS * 32, 5)
int4_gemv_kernel(const __grid_constant__ CUtensorMap tmW, int M, int N, int K, int group, const __half *__restrict__ act,
                 const __half *__restrict__ scales, __half *__restrict__ out, int *status)
{
    // The CTA's whole weight slab (16 rows x K/2 bytes) is requested from HBM at once: one tiled TMA load
    // per 256-k piece (a 16-row x 128-byte box, so the row stride is walked by the copy engine and a CTA
    // issues K/256 loads instead of hundreds of small row copies), one mbarrier per piece. Every byte the
    // kernel needs is in flight a few hundred cycles after the CTA starts, at no register cost. Each warp
    // owns a contiguous quarter of the pieces and computes on a piece as soon as it has landed, so the
    // work left after the last byte arrives is two 128-k blocks per warp.
    // kStageAct (M <= 2): the activations are additionally staged in shared memory, already permuted
    // to the slot order of the unpacked weights, which takes 16 byte-permutes and 4 global loads per
    // 128-k block out of the inner loop. For more rows that copy would not fit beside the weights.
    // Shared memory: [K/256 pieces][16 rows][128 B] weights | [16][G] fp16 scales | [mrows][K/8 + 1] uint4 staged
    // activations (kStageAct only).
    extern __shared__ __align__(128) uint8_t wsm[];
    __shared__ __align__(8) uint64_t bars[GEMV_MAX_PIECES];
    __shared__ float red[GEMV_WARPS * 16 * 8]; // cross-warp reduction [warp][16 rows][8 m]
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.y * 8;
    const int mrows = min(8, M - m0);
    const int n0 = blockIdx.x * GEMV_ROWS;
    const int nkb = K / 128;                                   // 128-k blocks per row
    const int npieces = (nkb + 1) / 2;                         // 256-k pieces per row
    const int ppw = (npieces + GEMV_WARPS - 1) / GEMV_WARPS;   // pieces per warp
    const int pc_lo = min(warp * ppw, npieces), pc_hi = min(pc_lo + ppw, npieces);
    const int G = K / group;
    const uint32_t wsm_u32 = (uint32_t)__cvta_generic_to_shared(wsm);
    const int w_bytes = npieces * GEMV_PIECE_BYTES;
    __half *sc_s = reinterpret_cast<__half *>(wsm + w_bytes);                 // [16][G]
    const int sc_bytes = (GEMV_ROWS * G * 2 + 15) & ~15;
    uint4 *act_s = reinterpret_cast<uint4 *>(wsm + w_bytes + sc_bytes);       // [mrows][act_pitch]
    const int act_pitch = K / 8 + 1; // uint4 per staged activation row (+1 keeps rows on different banks)

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < npieces; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&bars[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }

    // The small operands (scales, and the activations when they are staged) are requested BEFORE the
    // weight slab: a load issued after 22 MB of queued weight traffic would only come back once most of
    // that traffic has drained. They land in registers now and are written to shared memory after the
    // bulk copies have been issued.
    constexpr int SC_PRE = 4, ACT_PRE = 4; // per-thread prefetch depth; the rest (large K) is fetched afterwards
    const int sc_total = GEMV_ROWS * G, act_total = kStageAct ? mrows * (K / 8) : 0;
    __half sc_pre[SC_PRE];
    uint4 act_pre[ACT_PRE];
#pragma unroll
    for (int j = 0; j < SC_PRE; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        // The 16 rows' scales are one contiguous span of [N,G]; past the last row the index is clamped
        // (those rows are never stored).
        if (i < sc_total) sc_pre[j] = __ldg(scales + min((size_t)n0 * G + i, (size_t)N * G - 1));
    }
    __syncthreads(); // mbarriers initialised
    // One lane per piece: expect 2 KB on the piece's barrier and start its load. Rows past N and k past K
    // are zero-filled by the copy engine.
    if (lane < pc_hi - pc_lo) {
        const int pc = pc_lo + lane;
        const uint32_t bar = (uint32_t)__cvta_generic_to_shared(&bars[pc]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)GEMV_PIECE_BYTES) : "memory");
        tma_load_3d(wsm_u32 + (uint32_t)pc * GEMV_PIECE_BYTES, &tmW, pc * 128, n0, 0, bar);
    }
    // Programmatic dependent launch: weights and scales are constants, so everything above may run while
    // the previous kernel on the stream is still finishing. From here on this grid lets its own successor
    // start, and waits for its predecessor before touching the activations (which a predecessor may have
    // produced) or writing the output.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if constexpr (kStageAct) {
#pragma unroll
        for (int j = 0; j < ACT_PRE; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            // rows m0.. of act are contiguous: uint4 index i of the span
            if (i < act_total) act_pre[j] = __ldg(reinterpret_cast<const uint4 *>(act + (size_t)m0 * K) + i);
        }
    }
    // 8 consecutive activations -> {k0,k4}, {k1,k5}, {k2,k6}, {k3,k7}: the slot order of the unpacked weights
    auto permute8 = [](const uint4 &r) {
        uint4 o;
        o.x = __byte_perm(r.x, r.z, 0x5410);
        o.y = __byte_perm(r.x, r.z, 0x7632);
        o.z = __byte_perm(r.y, r.w, 0x5410);
        o.w = __byte_perm(r.y, r.w, 0x7632);
        return o;
    };
#pragma unroll
    for (int j = 0; j < SC_PRE; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < sc_total) sc_s[i] = sc_pre[j];
    }
    for (int i = threadIdx.x + SC_PRE * blockDim.x; i < sc_total; i += blockDim.x)
        sc_s[i] = __ldg(scales + min((size_t)n0 * G + i, (size_t)N * G - 1));
    if constexpr (kStageAct) {
#pragma unroll
        for (int j = 0; j < ACT_PRE; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            // at most two staged rows: the row index is a compare, not a division
            if (i < act_total) act_s[i + (i >= K / 8 ? 1 : 0)] = permute8(act_pre[j]);
        }
        for (int i = threadIdx.x + ACT_PRE * blockDim.x; i < act_total; i += blockDim.x)
            act_s[i + (i >= K / 8 ? 1 : 0)] = permute8(__ldg(reinterpret_cast<const uint4 *>(act + (size_t)m0 * K) + i));
    }
    __syncthreads(); // scales (and staged activations) visible to all warps
    const __half *sA = sc_s + g * G;
    const __half *sB = sc_s + (g + 8) * G;
    // Unstaged activations come straight from global memory: a few KB that every CTA on the SM reads, so
    // L1 hits after the first touch. Lane (g,t) supplies activation row g; lanes beyond the last row read
    // the last valid row (their output columns are never stored).
    const uint4 *arow = reinterpret_cast<const uint4 *>(act + (size_t)(m0 + min(g, mrows - 1)) * K) + t * 4;
    const int bpg = group / 128; // 128-k blocks per scale group
    const uint4 *arow_s = act_s + min(g, mrows - 1) * act_pitch + t * 4;
    const uint8_t *myA = wsm + g * 128 + t * 16;       // + piece * GEMV_PIECE_BYTES + (block in piece) * 64
    const uint8_t *myB = wsm + (g + 8) * 128 + t * 16;

    float tot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
    for (int pc = pc_lo; pc < pc_hi; ++pc) {
        if (!mbar_wait_warp((uint32_t)__cvta_generic_to_shared(&bars[pc]), 0u, &abort_flag, status, WAIT_EPI_STAGE)) break;
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
            const int kb = pc * 2 + blk;
            if (kb >= nkb) break;
            const uint4 qa = *reinterpret_cast<const uint4 *>(myA + pc * GEMV_PIECE_BYTES + blk * 64);
            const uint4 qb = *reinterpret_cast<const uint4 *>(myB + pc * GEMV_PIECE_BYTES + blk * 64);
            const uint32_t xa[4] = {qa.x, qa.y, qa.z, qa.w};
            const uint32_t xb[4] = {qb.x, qb.y, qb.z, qb.w};
            const int si = bpg == 1 ? kb : (int)((unsigned)kb / (unsigned)bpg);
            const float sa = __half2float(sA[si]);
            const float sb = __half2float(sB[si]);
            uint4 av[4];
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) av[wd] = kStageAct ? arow_s[kb * 16 + wd] : __ldg(arow + kb * 16 + wd);
            // Two independent accumulator chains halve the mma dependency depth.
            float c0[4], c1[4];
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
                uint32_t ha[4], hb[4];
                unpack8(xa[wd], ha);
                unpack8(xb[wd], hb);
                // 8 consecutive activations (k0..k7) -> the slot order of the unpacked weights:
                // {k0,k4}, {k1,k5}, {k2,k6}, {k3,k7}
                const uint32_t b04 = kStageAct ? av[wd].x : __byte_perm(av[wd].x, av[wd].z, 0x5410);
                const uint32_t b15 = kStageAct ? av[wd].y : __byte_perm(av[wd].x, av[wd].z, 0x7632);
                const uint32_t b26 = kStageAct ? av[wd].z : __byte_perm(av[wd].y, av[wd].w, 0x5410);
                const uint32_t b37 = kStageAct ? av[wd].w : __byte_perm(av[wd].y, av[wd].w, 0x7632);
                if (wd == 0) {
                    mma_16816_first(c0, ha[0], hb[0], ha[1], hb[1], b04, b15);
                    mma_16816_first(c1, ha[2], hb[2], ha[3], hb[3], b26, b37);
                } else {
                    mma_16816(c0, ha[0], hb[0], ha[1], hb[1], b04, b15);
                    mma_16816(c1, ha[2], hb[2], ha[3], hb[3], b26, b37);
                }
            }
            tot[0] = fmaf(sa, c0[0] + c1[0], tot[0]);
            tot[1] = fmaf(sa, c0[1] + c1[1], tot[1]);
            tot[2] = fmaf(sb, c0[2] + c1[2], tot[2]);
            tot[3] = fmaf(sb, c0[3] + c1[3], tot[3]);
        }
    }

    // Cross-warp reduction through shared memory.
    red[(warp * 16 + g) * 8 + 2 * t] = tot[0];
    red[(warp * 16 + g) * 8 + 2 * t + 1] = tot[1];
    red[(warp * 16 + g + 8) * 8 + 2 * t] = tot[2];
    red[(warp * 16 + g + 8) * 8 + 2 * t + 1] = tot[3];
    __syncthreads();
    if (abort_flag) {
        // A wait ran out: give copies still in flight a bounded time to land before the CTA's shared
        // memory is released, and store nothing.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
        return;
    }
    {
        const int m = threadIdx.x >> 4, r = threadIdx.x & 15; // 8 m x 16 rows = 128 threads
        float s = 0.f;
#pragma unroll
        for (int wi = 0; wi < GEMV_WARPS; ++wi) s += red[(wi * 16 + r) * 8 + m];
        if (m < mrows && n0 + r < N) out[(size_t)(m0 + m) * N + n0 + r] = __float2half_rn(s);
    }
}

// Shared-memory loads by 32-bit shared address with a compile-time byte offset: the inner loop of the streaming
// GEMV keeps one running address per operand and lets the offsets ride in the instruction.
template <int kOff>
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(kOff));
    return v;
}
__device__ __forceinline__ float lds_f16(uint32_t addr)
{
    unsigned short h;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(addr));
    return __half2float(__ushort_as_half(h));
}

// Streaming GEMV for M <= 8: one persistent CTA per SM walks the 16-row weight blocks c, c + grid, ... and
// keeps the weight stream running while it computes. A block's 16 rows are consecutive in memory (16 * K/2
// bytes, and its scales one span of 16 * G halves); a producer warp brings them in with bulk copies (one per
// row, so that the rows can be staged 64 bytes mod 128 apart: the lanes of one shared-memory access phase
// read two neighbouring rows) into one of two stages (full / empty mbarriers). Eight computing warps each
// own an eighth of K of every block and never meet on a CTA-wide barrier: a warp writes its partial sums,
// counts itself in, and the warp that arrives last adds the partials in warp order (so the result does not
// depend on arrival order) and stores the block's outputs.
// For M <= 4 the CTA uses less than half of an SM's shared memory and registers, and the grid is launched with
// programmatic stream serialisation: the next int4 launch on the stream becomes resident beside this one
// and streams its first blocks (weights and scales are parameters no predecessor writes) while this one is
// still computing; its computing warps touch the activations only after griddepcontrol.wait. Back-to-back
// launches (the layers of a decoder) therefore find their first blocks in shared memory when the predecessor
// ends, which the one-slab-per-CTA kernel above cannot offer: its CTAs hold all of shared memory until they
// exit.
// Measured (N = 11008, K = 4096, M = 1, launches back to back): 8.9 us per launch against 10.0 us for the slab
// kernel. Of that, 1.6 us pass between the predecessor's end and the return of griddepcontrol.wait, 0.5 us
// stage the activations, and each of a CTA's four or five blocks takes 1.1 us of arithmetic although its data
// is already in shared memory. That 1.1 us did not move with sixteen warps instead of eight, with half of the
// mma instructions or all of the fp16 offset removal taken out, or with a CTA barrier instead of the counter;
// packed-fp16 FMAs in place of the mma were slower (16.8 us).
constexpr int GS_WARPS = 8;  // computing warps; warp GS_WARPS is the producer
constexpr int GS_STAGES = 2; // weight blocks in flight per CTA
constexpr int GS_RED = 3;    // partial-sum buffers: a warp is never more than two blocks ahead of another

template <bool kStageAct>
__global__ void __launch_bounds__((GS_WARPS + 1) * 32, 2)
int4_gemv_stream_kernel(const uint8_t *__restrict__ w, int M, int N, int K, int group, const __half *__restrict__ act,
                        const __half *__restrict__ scales, __half *__restrict__ out, int *status)
{
    // Shared memory: GS_STAGES x ([16 rows][K/2 B] weights + [16][G] fp16 scales) | GS_RED x [8 warps][16 rows][mrows]
    // fp32 partials | [mrows][K/8 + 1] uint4 staged activations (kStageAct only).
    extern __shared__ __align__(128) uint8_t wsm[];
    __shared__ __align__(8) uint64_t bar_full[GS_STAGES], bar_empty[GS_STAGES];
    __shared__ int arrived[GS_RED];
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int mrows = min(8, M);
    const int nkb = K / 128;
    const int kpw = (nkb + GS_WARPS - 1) / GS_WARPS; // 128-k blocks per warp
    const int kb_lo = min(warp * kpw, nkb), kb_hi = min(kb_lo + kpw, nkb);
    const int G = K / group;
    const int row_bytes = K / 2;
    // Rows are staged 64 bytes (mod 128) apart: the eight lanes of one shared-memory access phase read two
    // neighbouring rows, which would otherwise fall on the same banks.
    const int row_pitch = row_bytes + ((192 - (row_bytes & 127)) & 127);
    const int w_bytes = GEMV_ROWS * row_pitch;
    const int stage_bytes = w_bytes + GEMV_ROWS * G * 2; // multiple of 16: G is a multiple of 8 on this path
    const int nblocks = (N + GEMV_ROWS - 1) / GEMV_ROWS;
    const int my_blocks = ((int)blockIdx.x < nblocks) ? (nblocks - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    float *red = reinterpret_cast<float *>(wsm + GS_STAGES * stage_bytes);
    const int red_floats = GS_WARPS * 16 * mrows;
    uint4 *act_s = reinterpret_cast<uint4 *>(wsm + GS_STAGES * stage_bytes + ((GS_RED * red_floats * 4 + 15) & ~15));
    const int act_pitch = K / 8 + 1;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < GS_RED; ++i) arrived[i] = 0;
        for (int i = 0; i < GS_STAGES; ++i) {
            mbar_init(smem_u32(&bar_full[i]), 1);
            mbar_init(smem_u32(&bar_empty[i]), GS_WARPS);
        }
        fence_mbar_init();
    }
    __syncthreads();
    // Programmatic dependent launch: this grid lets its successor start now. The producer never waits for the
    // predecessor (it reads weights and scales only); the computing warps do, before they read the activations
    // (which a predecessor may have produced) or write the output.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == GS_WARPS) {
        // ------------------------------------------------------------ producer: two bulk copies per block
        if (lane == 0) {
            for (int bi = 0; bi < my_blocks; ++bi) {
                const int stage = bi % GS_STAGES;
                if (bi >= GS_STAGES &&
                    !mbar_wait_short(smem_u32(&bar_empty[stage]), (uint32_t)((bi / GS_STAGES - 1) & 1), &abort_flag, status, WAIT_PRODUCER_EMPTY))
                    break;
                const int n0 = ((int)blockIdx.x + bi * (int)gridDim.x) * GEMV_ROWS;
                const int rows = min(GEMV_ROWS, N - n0); // rows past N are not read
                const uint32_t dst = smem_u32(wsm) + (uint32_t)stage * (uint32_t)stage_bytes;
                mbar_expect_tx(smem_u32(&bar_full[stage]), (uint32_t)(rows * (row_bytes + G * 2)));
                bulk_g2s(dst + (uint32_t)w_bytes, scales + (size_t)n0 * G, (uint32_t)(rows * G * 2), smem_u32(&bar_full[stage]));
                for (int r = 0; r < rows; ++r) // the rows are consecutive in memory: HBM still sees one sequential read
                    bulk_g2s(dst + (uint32_t)(r * row_pitch), w + (size_t)(n0 + r) * row_bytes, (uint32_t)row_bytes, smem_u32(&bar_full[stage]));
            }
        }
    } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if constexpr (kStageAct) {
            // 8 consecutive activations -> {k0,k4}, {k1,k5}, {k2,k6}, {k3,k7}: the slot order of the unpacked weights
            const int act_total = mrows * (K / 8);
            for (int i = threadIdx.x; i < act_total; i += GS_WARPS * 32) {
                const uint4 r = __ldg(reinterpret_cast<const uint4 *>(act) + i);
                uint4 o;
                o.x = __byte_perm(r.x, r.z, 0x5410);
                o.y = __byte_perm(r.x, r.z, 0x7632);
                o.z = __byte_perm(r.y, r.w, 0x5410);
                o.w = __byte_perm(r.y, r.w, 0x7632);
                act_s[i + i / (K / 8)] = o; // row pitch K/8 + 1: one pad word per row
            }
            asm volatile("bar.sync 1, 256;" ::: "memory"); // the computing warps' own barrier (GS_WARPS * 32 threads), once
        }
        // Lane (g, t) supplies activation row g to the mma's B operand; columns past the last row are never stored,
        // so their lanes load nothing (a shared-memory access with four active lanes is one wavefront, not four).
        const bool has_row = g < mrows;
        const uint4 *arow = reinterpret_cast<const uint4 *>(act + (size_t)min(g, mrows - 1) * K) + t * 4;
        const uint32_t act_u32 = smem_u32(act_s) + (uint32_t)((min(g, mrows - 1) * act_pitch + t * 4 + kb_lo * 16) * 16);
        const int bpg = group / 128;
        const uint32_t rowB_off = 8u * (uint32_t)row_pitch, sB_off = 16u * (uint32_t)G; // rows g + 8: weights, scales
        // Activation words of the lanes without a row stay zero for the whole kernel.
        uint4 av[4] = {make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u), make_uint4(0u, 0u, 0u, 0u)};

#pragma unroll 1
        for (int bi = 0; bi < my_blocks; ++bi) {
            const int stage = bi % GS_STAGES, slot = bi % GS_RED;
            const int n0 = ((int)blockIdx.x + bi * (int)gridDim.x) * GEMV_ROWS;
            float tot[4] = {0.f, 0.f, 0.f, 0.f};
            if (!mbar_wait_warp(smem_u32(&bar_full[stage]), (uint32_t)((bi / GS_STAGES) & 1), &abort_flag, status, WAIT_EPI_STAGE)) break;
            const uint32_t st_u32 = smem_u32(wsm) + (uint32_t)stage * (uint32_t)stage_bytes;
            uint32_t aW = st_u32 + (uint32_t)(g * row_pitch + t * 16 + kb_lo * 64);              // row g, this lane's 16 bytes of block kb
            const uint32_t aS0 = st_u32 + (uint32_t)w_bytes + (uint32_t)(g * G) * 2u;             // row g's scales
            uint32_t aA = act_u32;
#pragma unroll 1
            for (int kb = kb_lo; kb < kb_hi; ++kb, aW += 64u, aA += 256u) {
                const uint4 qa = lds128<0>(aW);
                const uint4 qb = lds128<0>(aW + rowB_off);
                const uint32_t xa[4] = {qa.x, qa.y, qa.z, qa.w};
                const uint32_t xb[4] = {qb.x, qb.y, qb.z, qb.w};
                const uint32_t aS = aS0 + 2u * (uint32_t)(bpg == 1 ? kb : (int)((unsigned)kb / (unsigned)bpg));
                const float sa = lds_f16(aS);
                const float sb = lds_f16(aS + sB_off);
                if (has_row) {
                    if constexpr (kStageAct) {
                        av[0] = lds128<0>(aA);
                        av[1] = lds128<16>(aA);
                        av[2] = lds128<32>(aA);
                        av[3] = lds128<48>(aA);
                    } else {
#pragma unroll
                        for (int wd = 0; wd < 4; ++wd) av[wd] = __ldg(arow + kb * 16 + wd);
                    }
                }
                float c0[4], c1[4];
#pragma unroll
                for (int wd = 0; wd < 4; ++wd) {
                    uint32_t ha[4], hb[4];
                    unpack8(xa[wd], ha);
                    unpack8(xb[wd], hb);
                    const uint32_t b04 = kStageAct ? av[wd].x : __byte_perm(av[wd].x, av[wd].z, 0x5410);
                    const uint32_t b15 = kStageAct ? av[wd].y : __byte_perm(av[wd].x, av[wd].z, 0x7632);
                    const uint32_t b26 = kStageAct ? av[wd].z : __byte_perm(av[wd].y, av[wd].w, 0x5410);
                    const uint32_t b37 = kStageAct ? av[wd].w : __byte_perm(av[wd].y, av[wd].w, 0x7632);
                    if (wd == 0) {
                        mma_16816_first(c0, ha[0], hb[0], ha[1], hb[1], b04, b15);
                        mma_16816_first(c1, ha[2], hb[2], ha[3], hb[3], b26, b37);
                    } else {
                        mma_16816(c0, ha[0], hb[0], ha[1], hb[1], b04, b15);
                        mma_16816(c1, ha[2], hb[2], ha[3], hb[3], b26, b37);
                    }
                }
                tot[0] = fmaf(sa, c0[0] + c1[0], tot[0]);
                tot[1] = fmaf(sa, c0[1] + c1[1], tot[1]);
                tot[2] = fmaf(sb, c0[2] + c1[2], tot[2]);
                tot[3] = fmaf(sb, c0[3] + c1[3], tot[3]);
            }
            // This warp's words and scales of the stage are consumed: hand the stage back.
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_empty[stage]));
            float *mine = red + slot * red_floats + warp * 16 * mrows;
            {
                // Partials [warp][row][m] of the valid activation rows; accumulator columns are m = 2t, 2t + 1.
                if (2 * t < mrows) {
                    mine[g * mrows + 2 * t] = tot[0];
                    mine[(g + 8) * mrows + 2 * t] = tot[2];
                }
                if (2 * t + 1 < mrows) {
                    mine[g * mrows + 2 * t + 1] = tot[1];
                    mine[(g + 8) * mrows + 2 * t + 1] = tot[3];
                }
            }
            __threadfence_block();
            __syncwarp();
            int last = 0;
            if (lane == 0) last = atomicAdd(&arrived[slot], 1) == GS_WARPS - 1;
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                __threadfence_block();
                // The last warp to arrive adds the partials in warp order and stores the block.
                for (int o = lane; o < 16 * mrows; o += 32) {
                    float sum = 0.f;
#pragma unroll
                    for (int wi = 0; wi < GS_WARPS; ++wi) sum += red[slot * red_floats + wi * 16 * mrows + o];
                    const int r = o / mrows, m = o - r * mrows;
                    if (n0 + r < N) out[(size_t)m * N + n0 + r] = __float2half_rn(sum);
                }
                __syncwarp();
                if (lane == 0) arrived[slot] = 0; // reused three blocks on, after every warp has passed this block
            }
        }
    }
    __syncthreads();
    if (abort_flag) {
        // A wait ran out: give copies still in flight a bounded time to land before the CTA's shared
        // memory is released.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
    }
}

// Eight nibbles of one word -> four half2 in NATURAL pair order {k0,k1}, {k2,k3}, {k4,k5}, {k6,k7}, so that
// activations can be used as they lie in memory. A byte-permute puts each byte in both halves of a word;
// (x & 0x00F0000F) ^ 0x64806408 then makes {1032 + v_even, 1152 + 16 v_odd} and one HFMA2 with per-half
// constants {1, 1/16} and {-1032, -72} removes the offsets exactly.
__device__ __forceinline__ void unpack8_natural(uint32_t x, uint32_t (&h)[4])
{
    const __half2 mul = __halves2half2(__ushort_as_half((unsigned short)0x3C00), __ushort_as_half((unsigned short)0x2C00)); // {1, 1/16}
    const __half2 add = __halves2half2(__ushort_as_half((unsigned short)0xE408), __ushort_as_half((unsigned short)0xD480)); // {-1032, -72}
    const uint32_t y = __byte_perm(x, x, 0x1010); // bytes b0 b1 b0 b1
    const uint32_t z = __byte_perm(x, x, 0x3232); // bytes b2 b3 b2 b3
    uint32_t p01 = and_xor(y, 0x00F0000Fu, 0x64806408u);
    uint32_t p23 = and_xor(y >> 8, 0x00F0000Fu, 0x64806408u);
    uint32_t p45 = and_xor(z, 0x00F0000Fu, 0x64806408u);
    uint32_t p67 = and_xor(z >> 8, 0x00F0000Fu, 0x64806408u);
    __half2 r0 = __hfma2(*reinterpret_cast<__half2 *>(&p01), mul, add);
    __half2 r1 = __hfma2(*reinterpret_cast<__half2 *>(&p23), mul, add);
    __half2 r2 = __hfma2(*reinterpret_cast<__half2 *>(&p45), mul, add);
    __half2 r3 = __hfma2(*reinterpret_cast<__half2 *>(&p67), mul, add);
    h[0] = *reinterpret_cast<uint32_t *>(&r0);
    h[1] = *reinterpret_cast<uint32_t *>(&r1);
    h[2] = *reinterpret_cast<uint32_t *>(&r2);
    h[3] = *reinterpret_cast<uint32_t *>(&r3);
}

// int4 matmul for 8 < M <= 64 per launch row-group: the structure of int4_gemv_kernel (weight slab
// staged once with bulk copies, 16 weight rows per CTA, K split over 4 warps), but every unpacked
// weight block is reused for MB activation row-blocks of 8, so the weights are read from HBM and
// unpacked once for up to 64 rows. Activations are read in natural order from global memory (L1/L2).
template <int MB>
__global__ void __launch_bounds__(GEMV_WARPS * 32, 4)
int4_gemm_mma_kernel(int M, int N, int K, int group, const __half *__restrict__ act, const uint8_t *__restrict__ w,
                     const __half *__restrict__ scales, __half *__restrict__ out, int *status)
{
    extern __shared__ __align__(128) uint8_t wsm[]; // [16][K/2 + GEMV_ROW_PAD] weights | [16][G] scales | reduction buffer
    __shared__ __align__(8) uint64_t bars[GEMV_WARPS * 2];
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.y * (8 * MB);
    const int mrows = min(8 * MB, M - m0);
    const int n0 = blockIdx.x * GEMV_ROWS;
    const int nkb = K / 128;
    const int bpw = (nkb + GEMV_WARPS - 1) / GEMV_WARPS;
    const int kb_lo = min(warp * bpw, nkb), kb_hi = min(kb_lo + bpw, nkb);
    const int kb_mid = kb_lo + (kb_hi - kb_lo + 1) / 2;
    const int G = K / group;
    const int row_bytes = K / 2;
    const int row_pitch = row_bytes + GEMV_ROW_PAD;
    const uint32_t wsm_u32 = (uint32_t)__cvta_generic_to_shared(wsm);
    __half *sc_s = reinterpret_cast<__half *>(wsm + GEMV_ROWS * row_pitch);
    const int sc_bytes = (GEMV_ROWS * G * 2 + 15) & ~15;
    float *red = reinterpret_cast<float *>(wsm + GEMV_ROWS * row_pitch + sc_bytes); // [warp][16 rows][8*MB]

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < GEMV_WARPS * 2; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"((uint32_t)__cvta_generic_to_shared(&bars[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Scales first (see int4_gemv_kernel: small loads queued behind the weight slab would return last).
    constexpr int SC_PRE = 4;
    const int sc_total = GEMV_ROWS * G;
    __half sc_pre[SC_PRE];
#pragma unroll
    for (int j = 0; j < SC_PRE; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < sc_total) sc_pre[j] = __ldg(scales + min((size_t)n0 * G + i, (size_t)N * G - 1));
    }
    __syncthreads();
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(&bars[warp * 2]);
    const uint32_t bar1 = bar0 + 8;
    {
        const uint32_t bytes0 = (uint32_t)(kb_mid - kb_lo) * 64u, bytes1 = (uint32_t)(kb_hi - kb_mid) * 64u;
        if (lane == 0) {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar0), "r"(bytes0 * 16u) : "memory");
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar1), "r"(bytes1 * 16u) : "memory");
        }
        __syncwarp();
        if (lane < GEMV_ROWS) {
            const int row = min(n0 + lane, N - 1);
            const uint8_t *src = w + (size_t)row * row_bytes;
            const uint32_t dst = wsm_u32 + (uint32_t)(lane * row_pitch);
            if (bytes0) bulk_g2s(dst + kb_lo * 64, src + kb_lo * 64, bytes0, bar0);
            if (bytes1) bulk_g2s(dst + kb_mid * 64, src + kb_mid * 64, bytes1, bar1);
        }
    }
#pragma unroll
    for (int j = 0; j < SC_PRE; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < sc_total) sc_s[i] = sc_pre[j];
    }
    for (int i = threadIdx.x + SC_PRE * blockDim.x; i < sc_total; i += blockDim.x)
        sc_s[i] = __ldg(scales + min((size_t)n0 * G + i, (size_t)N * G - 1));
    __syncthreads();
    const __half *sA = sc_s + g * G;
    const __half *sB = sc_s + (g + 8) * G;
    const int bpg = group / 128;
    const uint8_t *myA = wsm + g * row_pitch + t * 16;
    const uint8_t *myB = wsm + (g + 8) * row_pitch + t * 16;
    // Activation row of this lane in row-block j: m0 + 8 j + g, clamped (columns past M are never stored).
    const uint4 *abase = reinterpret_cast<const uint4 *>(act) + t * 4;

    float tot[MB][4];
#pragma unroll
    for (int j = 0; j < MB; ++j) tot[j][0] = tot[j][1] = tot[j][2] = tot[j][3] = 0.f;
    bool ok = true;
#pragma unroll 1
    for (int half = 0; half < 2 && ok; ++half) {
        const int b0 = half ? kb_mid : kb_lo, b1 = half ? kb_hi : kb_mid;
        if (b0 >= b1) continue;
        ok = mbar_wait_warp(half ? bar1 : bar0, 0u, &abort_flag, status, WAIT_EPI_STAGE);
        if (!ok) break;
#pragma unroll 1
        for (int kb = b0; kb < b1; ++kb) {
            const uint4 qa = *reinterpret_cast<const uint4 *>(myA + kb * 64);
            const uint4 qb = *reinterpret_cast<const uint4 *>(myB + kb * 64);
            const uint32_t xa[4] = {qa.x, qa.y, qa.z, qa.w};
            const uint32_t xb[4] = {qb.x, qb.y, qb.z, qb.w};
            uint32_t ha[4][4], hb[4][4];
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
                unpack8_natural(xa[wd], ha[wd]);
                unpack8_natural(xb[wd], hb[wd]);
            }
            const int si = bpg == 1 ? kb : (int)((unsigned)kb / (unsigned)bpg);
            const float sa = __half2float(sA[si]);
            const float sb = __half2float(sB[si]);
#pragma unroll
            for (int j = 0; j < MB; ++j) {
                const int m = m0 + min(8 * j + g, mrows - 1);
                const uint4 *arow = abase + (size_t)m * (K / 8) + kb * 16;
                uint4 av[4];
#pragma unroll
                for (int wd = 0; wd < 4; ++wd) av[wd] = __ldg(arow + wd);
                float c0[4], c1[4];
#pragma unroll
                for (int wd = 0; wd < 4; ++wd) {
                    if (wd == 0) {
                        mma_16816_first(c0, ha[wd][0], hb[wd][0], ha[wd][1], hb[wd][1], av[wd].x, av[wd].y);
                        mma_16816_first(c1, ha[wd][2], hb[wd][2], ha[wd][3], hb[wd][3], av[wd].z, av[wd].w);
                    } else {
                        mma_16816(c0, ha[wd][0], hb[wd][0], ha[wd][1], hb[wd][1], av[wd].x, av[wd].y);
                        mma_16816(c1, ha[wd][2], hb[wd][2], ha[wd][3], hb[wd][3], av[wd].z, av[wd].w);
                    }
                }
                tot[j][0] = fmaf(sa, c0[0] + c1[0], tot[j][0]);
                tot[j][1] = fmaf(sa, c0[1] + c1[1], tot[j][1]);
                tot[j][2] = fmaf(sb, c0[2] + c1[2], tot[j][2]);
                tot[j][3] = fmaf(sb, c0[3] + c1[3], tot[j][3]);
            }
        }
    }

    // Cross-warp reduction: red[warp][row 0..15][m 0..8*MB)
    constexpr int MW = 8 * MB;
#pragma unroll
    for (int j = 0; j < MB; ++j) {
        red[(warp * 16 + g) * MW + 8 * j + 2 * t] = tot[j][0];
        red[(warp * 16 + g) * MW + 8 * j + 2 * t + 1] = tot[j][1];
        red[(warp * 16 + g + 8) * MW + 8 * j + 2 * t] = tot[j][2];
        red[(warp * 16 + g + 8) * MW + 8 * j + 2 * t + 1] = tot[j][3];
    }
    __syncthreads();
    if (abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
        return;
    }
    for (int i = threadIdx.x; i < 16 * MW; i += blockDim.x) {
        const int m = i >> 4, r = i & 15; // consecutive threads -> consecutive output columns
        float sacc = 0.f;
#pragma unroll
        for (int wi = 0; wi < GEMV_WARPS; ++wi) sacc += red[(wi * 16 + r) * MW + m];
        if (m < mrows && n0 + r < N) out[(size_t)(m0 + m) * N + n0 + r] = __float2half_rn(sacc);
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
    // One thread per packed 32-bit word (8 weights) -> one 16-byte store; a warp reads 128 and writes 512 contiguous
    // bytes. Word i lies in row i / (K/8) at k = 8 * (i mod (K/8)); 8 divides the group, so one scale per word.
    const long long words = nbytes / 4;
    const int G = K / group;
    const uint32_t wpr = (uint32_t)K >> 3, gshift_words = (uint32_t)group >> 3; // words per row, words per group
    const bool small = words <= 0xFFFFFFFFLL;
    const long long stride = (long long)gridDim.x * blockDim.x;
    constexpr int UN = 4; // words in flight per thread: one load per thread at a time left the read side latency-bound
    for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < words; i0 += UN * stride) {
        uint32_t x[UN];
        __half sc[UN];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const long long i = i0 + u * stride;
            if (i < words) {
                x[u] = __ldg(reinterpret_cast<const uint32_t *>(w) + i);
                long long n;
                uint32_t wi; // word index inside the row
                if (small) { // 32-bit division: the 64-bit one costs more than the rest of the thread's work
                    const uint32_t q = (uint32_t)i / wpr;
                    n = q;
                    wi = (uint32_t)i - q * wpr;
                } else {
                    n = i / wpr;
                    wi = (uint32_t)(i - n * wpr);
                }
                sc[u] = __ldg(scales + n * G + wi / gshift_words);
            }
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const long long i = i0 + u * stride;
            if (i < words) reinterpret_cast<uint4 *>(out)[i] = dequant_word(x[u], __half2half2(sc[u]));
        }
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

int configure_int4_gemv_kernels()
{
    cudaError_t e = cudaFuncSetAttribute(int4_gemv_stream_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 150 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(int4_gemv_stream_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 150 * 1024);
    int rc = check_cuda(e, "cudaFuncSetAttribute(int4_gemv_stream)");
    if (rc) return rc;
    return configure_int4_gemv_regs_kernels();
}

int launch_int4_gemv(cudaStream_t st, int sm_count, int M, int N, int K, int group, const void *act, const void *w,
                     const void *scales, void *out, int *status)
{
    if (M == 0 || N == 0) return BTM_OK;
    const bool fast = (K % 128 == 0) && (group % 128 == 0) && (((uintptr_t)act & 15) == 0) && (((uintptr_t)w & 15) == 0) &&
                      (((uintptr_t)scales & 1) == 0) && K > 0 && (size_t)GEMV_ROWS * (K / 2 + GEMV_ROW_PAD + 2 * (K / group)) + 2 * (size_t)(K / 8 + 1) * 16 <= 200 * 1024;
    if (!fast) {
        const long long total = (long long)M * N;
        const int block = 128;
        const long long grid = (total + block - 1) / block;
        if (grid > 0x7FFFFFFFLL) return set_error(BTM_ERR_UNSUPPORTED, "int4 matmul: output too large");
        int4_matmul_general_kernel<<<(unsigned)grid, block, 0, st>>>(M, N, K, group, (const __half *)act, (const uint8_t *)w,
                                                                     (const __half *)scales, (__half *)out);
        return check_cuda(cudaGetLastError(), "int4 general launch");
    }
    if (M > 8) {
        // Several activation row-blocks per CTA: weights are fetched and unpacked once for up to 64 rows.
        const int mb = M <= 16 ? 2 : (M <= 32 ? 4 : 8);
        const size_t smem_mb = (size_t)GEMV_ROWS * (K / 2 + GEMV_ROW_PAD) + (((size_t)GEMV_ROWS * (K / group) * 2 + 15) & ~(size_t)15) +
                               (size_t)GEMV_WARPS * 16 * 8 * mb * sizeof(float);
        dim3 grid_mb((unsigned)((N + GEMV_ROWS - 1) / GEMV_ROWS), (unsigned)((M + 8 * mb - 1) / (8 * mb)));
        cudaError_t e = cudaSuccess;
#define BTM_LAUNCH_MB(MBV)                                                                                                        \
    do {                                                                                                                          \
        if (smem_mb > 48 * 1024)                                                                                                  \
            e = cudaFuncSetAttribute(int4_gemm_mma_kernel<MBV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);         \
        if (e == cudaSuccess)                                                                                                     \
            int4_gemm_mma_kernel<MBV><<<grid_mb, GEMV_WARPS * 32, smem_mb, st>>>(M, N, K, group, (const __half *)act,             \
                                                                                 (const uint8_t *)w, (const __half *)scales,      \
                                                                                 (__half *)out, status);                          \
    } while (0)
        if (mb == 2) BTM_LAUNCH_MB(2);
        else if (mb == 4) BTM_LAUNCH_MB(4);
        else BTM_LAUNCH_MB(8);
#undef BTM_LAUNCH_MB
        int rc = check_cuda(e, "cudaFuncSetAttribute(int4_gemm_mma)");
        if (rc) return rc;
        return check_cuda(cudaGetLastError(), "int4 gemm launch");
    }
    // M <= 8: the register-resident kernel (int4_gemv_regs.cu) wherever it takes the shape. On the 11008 x 4096 workload
    // it runs 7.1 / 7.6 / 8.5 / 9.9 us at M = 1 / 2 / 4 / 8 against 9.1 / 9.2 / 9.4 / 11.0 us for the streaming kernel
    // below. BTM_FORCE_GEMV=regs|stream|slab pins a kernel (the tests use it to run every kernel on every shape it
    // takes). Shapes a kernel does not take fall through to the next.
    const char *force_gemv = getenv("BTM_FORCE_GEMV");
    const bool want_regs = force_gemv ? !strcmp(force_gemv, "regs") : true;
    if (want_regs) {
        const int rc_regs = launch_int4_gemv_regs(st, sm_count, M, N, K, group, act, w, scales, out);
        if (rc_regs != -1) return rc_regs;
    }
    const bool stage_act = M <= 2; // slab kernel: a slab and more than two staged rows do not fit together
    const int npieces = (K / 128 + 1) / 2;
    // Streaming kernel: K long enough to give each of its eight warps a 128-k block, a block's scales a whole
    // number of 16-byte units at a 16-byte-aligned address, and two stages plus the partial sums within its shared
    // memory budget. The activations are staged beside them when that still fits: up to 110 KB in all for M <= 4
    // (the next launch then fits on the SM beside this one), up to 150 KB for more rows (13.1 -> 10.9 us at M = 8:
    // the permuted copy takes four global loads and eight byte-permutes per 128-k block out of the inner loop,
    // which is worth more there than the early residency of the successor).
    const int mrows_s = M < 8 ? M : 8;
    const size_t smem_base_s = (size_t)GS_STAGES * GEMV_ROWS * (K / 2 + ((192 - ((K / 2) & 127)) & 127) + (K / group) * 2) +
                               (((size_t)GS_RED * GS_WARPS * 16 * mrows_s * 4 + 15) & ~(size_t)15);
    const size_t smem_staged = smem_base_s + (size_t)M * (K / 8 + 1) * sizeof(uint4);
    const bool stage_act_stream = smem_staged <= (size_t)(M <= 4 ? 110 : 150) * 1024;
    const size_t smem_stream = stage_act_stream ? smem_staged : smem_base_s;
    const bool stream_ok = K / 128 >= GS_WARPS && (K / 2) % 16 == 0 && (K / group) % 8 == 0 && (((uintptr_t)scales & 15) == 0) &&
                           smem_stream <= 150 * 1024 && !(force_gemv && !strcmp(force_gemv, "slab"));
    if (stream_ok) {
        const void *fn = stage_act_stream ? (const void *)int4_gemv_stream_kernel<true> : (const void *)int4_gemv_stream_kernel<false>;
        const int nblocks = (N + GEMV_ROWS - 1) / GEMV_ROWS;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(nblocks < sm_count ? nblocks : sm_count));
        cfg.blockDim = dim3((GS_WARPS + 1) * 32);
        cfg.dynamicSmemBytes = smem_stream;
        cfg.stream = st;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization; // the kernel orders itself with griddepcontrol
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        const __half *act_h = (const __half *)act, *sc_h = (const __half *)scales;
        const uint8_t *w_b = (const uint8_t *)w;
        __half *out_h = (__half *)out;
        void *args[] = {(void *)&w_b, (void *)&M, (void *)&N, (void *)&K, (void *)&group, (void *)&act_h, (void *)&sc_h, (void *)&out_h, (void *)&status};
        cudaError_t le = cudaLaunchKernelExC(&cfg, fn, args);
        if (le != cudaSuccess) return check_cuda(le, "int4 gemv launch");
        return check_cuda(cudaGetLastError(), "int4 gemv launch");
    }
    dim3 grid((unsigned)((N + GEMV_ROWS - 1) / GEMV_ROWS), (unsigned)((M + 7) / 8));
    if (npieces > GEMV_MAX_PIECES) return set_error(BTM_ERR_UNSUPPORTED, "int4 matmul: K=%d is beyond the fast kernel's limit of %d", K, GEMV_MAX_PIECES * 256);
    CUtensorMap tmW;
    int rc = encode_tmap_3d(&tmW, BTM_U8, w, (uint64_t)K / 2, (uint64_t)N, 1, (uint64_t)K / 2, (uint64_t)K / 2, 128, GEMV_ROWS, false);
    if (rc) return rc;
    size_t smem = (size_t)npieces * GEMV_PIECE_BYTES + (((size_t)GEMV_ROWS * (K / group) * 2 + 15) & ~(size_t)15);
    if (stage_act) smem += (size_t)M * (K / 8 + 1) * sizeof(uint4);
    if (smem > 48 * 1024) {
        cudaError_t e = stage_act ? cudaFuncSetAttribute(int4_gemv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)
                                  : cudaFuncSetAttribute(int4_gemv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        rc = check_cuda(e, "cudaFuncSetAttribute(int4_gemv)");
        if (rc) return rc;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(GEMV_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization; // the kernel orders itself with griddepcontrol
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const __half *act_h = (const __half *)act, *sc_h = (const __half *)scales;
    __half *out_h = (__half *)out;
    cudaError_t le = stage_act ? cudaLaunchKernelEx(&cfg, int4_gemv_kernel<true>, tmW, M, N, K, group, act_h, sc_h, out_h, status)
                               : cudaLaunchKernelEx(&cfg, int4_gemv_kernel<false>, tmW, M, N, K, group, act_h, sc_h, out_h, status);
    if (le != cudaSuccess) return check_cuda(le, "int4 gemv launch");
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
