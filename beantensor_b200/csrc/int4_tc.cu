// int4 weight-only matmul on the tensor cores for 8 < M <= 128 rows per pass:
//   out[m, n] = sum_k act[m, k] * dq[n, k],   dq[n, k] = f16_rne(float(W[n, k]) * float(S[n, k / group]))
// i.e. the weights are dequantised exactly as btm_int4_dequant defines them and the product runs as an
// fp16 tcgen05 matmul with fp32 accumulation in tensor memory.
//
// The product is computed transposed: the 128 dequantised weight rows of a CTA are the tensor core's
// A operand (its full 128-row datapath), the activation rows are the B operand (UMMA N = the rows of the
// pass rounded up to 16), so no tensor-core row is spent on padding when M is small. K is split over the CTAs of a cluster, which
// puts two or three times as many CTAs on the machine as there are 128-row weight tiles (86 for
// N = 11008) and divides the activation bytes a CTA pulls from L2 by the same factor; the partial
// accumulators are summed over the cluster's shared memory, every CTA taking a share of the activation rows.
//
// Roles in a CTA (11 warps), per 128-k unit of its K slice:
//   warp 0      TMA: packed weights, 128 rows x 64 B (64-byte swizzle), ring of 4-6 units;
//   warp 2      TMA: activation tiles, MB rows x 64 k (K-major, 128-byte swizzle), two per unit, in a stage that
//               is tied to the unit's stage in tensor memory (filled and freed together);
//   warps 3-10  dequantise: thread = weight row, the two groups of four warps take alternate units; four
//               128-bit shared loads, unpack to exact fp16 integers in natural k order, multiply by
//               the group scale, and write the row's 128 fp16 straight into tensor memory (tcgen05.st,
//               64 columns of the thread's own lane): the tensor core takes its A operand from
//               there, so the tile never passes through shared memory and needs no proxy fence. A
//               warp passes one set of hand-offs per 128 k. The unpack instructions of these warps
//               are what the main loop's time is made of (24 issue cycles per 32-bit word);
//   warp 1      tcgen05.mma (M = 128, N = MB, A from tensor memory, B K-major in shared memory): one wait,
//               eight MMAs and one tcgen05.commit per unit (the commit frees the unit in tensor memory and
//               its activations). Its issue is serial and shares the tensor pipe with the SM's other CTA,
//               so everything else has been moved off this warp, and it walks its loop as a whole warp with
//               warp-uniform descriptors (one elected lane issues).
// Then every CTA parks its accumulator (lane = weight row, column = activation row) in its own shared
// memory, and after one cluster barrier CTA r fetches block r of the columns from all CTAs over DSMEM,
// adds them in rank order, rounds once to fp16, transposes through shared memory and stores rows of 256
// contiguous bytes of out[m, n0 .. n0 + 128) for its block of m.
// The kernel is launched with programmatic stream serialisation: weights and scales are fetched while the
// predecessor on the stream may still run; activations are read and the output written after griddepcontrol.wait.
// HBM traffic: the packed weights once (N*K/2 bytes) plus scales; activations come from L2
// (N/128 x M x K x 2 bytes in total, whatever the split).
#include <cuda_fp16.h>

#include "btm_internal.h"
#include "btm_ptx.cuh"
#include "int4_unpack.cuh"

namespace btm {

namespace i4tc {
constexpr int BW = 128;            // weight rows per CTA = UMMA M
constexpr int BKE = 64;            // k per operand stage
constexpr int UNIT_K = 128;        // k per raw-weight unit (64 bytes per row)
constexpr int RAW_BYTES = BW * 64; // 8 KB
constexpr int W_COLS = 64;         // dequantised unit in tensor memory: 128 lanes x 64 columns = 128 rows x 128 k fp16
constexpr int TMEM_COLS = 256;     // accumulator (MB columns) + ring of dequantised tiles
constexpr int THREADS = 352;       // warp 0 weight TMA, 1 MMA, 2 activation TMA, 3..10 dequantise + epilogue
constexpr int DQ_FIRST = 96;       // first dequantising thread
constexpr int MAX_SPLIT = 3;
template <int MB> // activation rows per pass: 64 or 128 (= UMMA N = accumulator columns)
struct Cfg {
    static constexpr int RAW_STAGES = MB == 64 ? 6 : 4;
    static constexpr int W_STAGES = (TMEM_COLS - MB) / W_COLS; // 3 or 2 units in tensor memory
    static constexpr int ACT_STAGES = W_STAGES;                // one activation stage (128 k) per unit in tensor memory
    static constexpr int ACT_HALF = MB * 128;                  // one 64-k block: MB rows of 128 bytes
    static constexpr int ACT_BYTES = 2 * ACT_HALF;
    static constexpr int RING_BYTES = ACT_STAGES * ACT_BYTES + RAW_STAGES * RAW_BYTES;
    // After the main loop the rings are dead and hold the parked accumulator (MB x 128 fp32) and behind it the output tile.
    static_assert(MB * BW * 4 + MB * BW * 2 <= RING_BYTES, "parked accumulator and output tile must fit in the rings");
    static constexpr int SMEM_BYTES = RING_BYTES + 1024; // + BW * groups-in-slice * 2 bytes of scales at run time
};
constexpr int SCALE_SMEM_MAX = 6144;
} // namespace i4tc

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_ctaid_x()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
// All threads of all CTAs of the cluster; release/acquire, so shared-memory stores made before it (also
// into another CTA's shared memory) are visible after it.
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
    return r;
}
template <int MB>
__global__ void __launch_bounds__(i4tc::THREADS, 2)
int4_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmAct, const __grid_constant__ CUtensorMap tmW, const GemmParams p,
                    const __half *__restrict__ scales, int group, int m_base, int n_inst)
{
    using namespace i4tc;
    using C = Cfg<MB>;
    constexpr int RAW_STAGES = C::RAW_STAGES, ACT_STAGES = C::ACT_STAGES, W_STAGES = C::W_STAGES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_raw_full[RAW_STAGES], bar_raw_empty[RAW_STAGES];
    __shared__ __align__(8) uint64_t bar_act_full[ACT_STAGES], bar_w_full[W_STAGES], bar_w_empty[W_STAGES];
    __shared__ __align__(8) uint64_t bar_acc_full;
    __shared__ uint32_t tmem_base_holder;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t act_ring = smem_base;
    const uint32_t raw_ring = act_ring + ACT_STAGES * C::ACT_BYTES;
    __half *sc_s = reinterpret_cast<__half *>(smem_al + C::RING_BYTES);

    const uint32_t crank = cluster_ctarank(), csize = cluster_nctarank();
    const int tile = (int)cluster_ctaid_x();
    const int n0 = tile * BW;
    // This CTA's K slice, in 128-k units; every CTA starts its walk at a different unit of the slice: CTAs of
    // the same rank read the same activations and in lock step would all ask the same L2 lines at once.
    // (Everything here is on every thread's way to its first useful instruction: 32-bit unsigned divisions only.)
    const uint32_t ugroup = (uint32_t)group;
    const int units = p.K / UNIT_K;
    const int u0 = (int)((uint32_t)units * crank / csize), u1 = (int)((uint32_t)units * (crank + 1u) / csize);
    const int n_units = u1 - u0;
    const int u_first = n_units > 0 ? (int)((uint32_t)tile % (uint32_t)n_units) : 0;
    const int g_first = (int)((uint32_t)(u0 * UNIT_K) / ugroup);
    const int g_cnt = n_units > 0 ? (int)((uint32_t)(u1 * UNIT_K - 1) / ugroup) - g_first + 1 : 0;
    // i-th unit of this CTA's walk
    auto unit_at = [&](int i) {
        int u = u_first + i;
        if (u >= n_units) u -= n_units;
        return u + u0;
    };

    // Programmatic dependent launch: this grid lets its successor on the stream start as soon as the machine has
    // room for its CTAs. Weights and scales are constants, so a CTA may fetch them while its predecessor still runs;
    // the activations are read and the output is written only after griddepcontrol.wait (warp 2 and the epilogue).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0 && lane == 0) {
        // The first weight units are requested before anything else in the CTA is set up: they come from HBM
        // and everything downstream waits for them.
        for (int i = 0; i < RAW_STAGES; ++i) mbar_init(smem_u32(&bar_raw_full[i]), 1);
        fence_mbar_init();
        for (int i = 0; i < RAW_STAGES && i < n_units; ++i) {
            mbar_expect_tx(smem_u32(&bar_raw_full[i]), RAW_BYTES);
            tma_load_3d(raw_ring + i * RAW_BYTES, &tmW, unit_at(i) * (UNIT_K / 2), n0, 0, smem_u32(&bar_raw_full[i]));
        }
        abort_flag = 0;
        for (int i = 0; i < RAW_STAGES; ++i) mbar_init(smem_u32(&bar_raw_empty[i]), 4);
        for (int i = 0; i < W_STAGES; ++i) {
            mbar_init(smem_u32(&bar_act_full[i]), 1);
            mbar_init(smem_u32(&bar_w_full[i]), 4);
            mbar_init(smem_u32(&bar_w_empty[i]), 1);
        }
        mbar_init(smem_u32(&bar_acc_full), 1);
        fence_mbar_init();
    }
    // The dequantising warps ask for their slice's scales before anything else happens in the CTA: once the weight
    // ring's first loads are queued (a dozen megabytes over the whole grid) a small load comes back microseconds
    // later, and no weight can be dequantised before the scales are there.
    constexpr int SC_PRE = 6; // per-thread prefetch depth; the rest (long K or small groups) is fetched afterwards
    __half sc_pre[SC_PRE];
    const int sc_total = BW * g_cnt, G = (int)((uint32_t)p.K / ugroup);
#ifndef BTM_I4TC_SCALES_DIRECT
#define BTM_I4TC_SCALES_DIRECT 0
#endif
    // Direct form: a dequantising thread (= weight row) fetches the two scales of a unit from global memory one unit
    // ahead of their use, so nothing is staged and the eight warps do not meet before their first unit.
    __half sd0 = __ushort_as_half((unsigned short)0), sd1 = sd0;
    if (BTM_I4TC_SCALES_DIRECT && warp >= 3 && n_units > 0) {
        const int grp0 = (warp - 3) >> 2, row0 = (warp & 3) * 32 + lane;
        if (grp0 < n_units) {
            const int u = unit_at(grp0);
            const __half *grow = scales + (size_t)min(n0 + row0, p.N - 1) * G;
            sd0 = __ldg(grow + (u * UNIT_K) / group);
            sd1 = __ldg(grow + (u * UNIT_K + BKE) / group);
        }
    }
    if (!BTM_I4TC_SCALES_DIRECT && warp >= 3 && g_cnt > 0) {
        // element i = r * g_cnt + g of the slice's scales; one division, then steps of 256 elements
        const uint32_t i0 = threadIdx.x - DQ_FIRST, gc = (uint32_t)g_cnt, rstep = 256u / gc, gstep = 256u - rstep * gc;
        uint32_t r = i0 / gc, g = i0 - r * gc;
#pragma unroll
        for (int j = 0; j < SC_PRE; ++j) {
            if ((int)i0 + j * 256 < sc_total) sc_pre[j] = __ldg(scales + (size_t)min(n0 + (int)r, p.N - 1) * G + g_first + (int)g);
            r += rstep;
            g += gstep;
            if (g >= gc) { g -= gc; ++r; }
        }
    }

    if (warp == 1) {
        tmem_alloc<1>(smem_u32(&tmem_base_holder), TMEM_COLS);
        tmem_relinquish<1>();
    }
    if (warp == 2 && lane == 0) prefetch_tmap(&tmAct);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_holder;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer: packed weights
        if (lane == 0) {
            int rs = 0;
            uint32_t rphase = 1; // the ring was filled once during set-up
            for (int i = RAW_STAGES; i < n_units; ++i) {
                if (!mbar_wait(smem_u32(&bar_raw_empty[rs]), rphase ^ 1u, &abort_flag, p.status, WAIT_PRODUCER_EMPTY)) break;
                mbar_expect_tx(smem_u32(&bar_raw_full[rs]), RAW_BYTES);
                tma_load_3d(raw_ring + rs * RAW_BYTES, &tmW, unit_at(i) * (UNIT_K / 2), n0, 0, smem_u32(&bar_raw_full[rs]));
                if (++rs == RAW_STAGES) { rs = 0; rphase ^= 1u; }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------ TMA producer: activation tiles
        if (lane == 0) {
            // Stage ws of the activations lives and dies with stage ws of the unpacked weights: the commit that
            // frees the unit in tensor memory (bar_w_empty) frees its activations too.
            int as = 0;
            uint32_t aphase = 0;
            asm volatile("griddepcontrol.wait;" ::: "memory"); // the activations may be the predecessor's output
            for (int i = 0; i < n_units; ++i) {
                const int u = unit_at(i);
                if (!mbar_wait(smem_u32(&bar_w_empty[as]), aphase ^ 1u, &abort_flag, p.status, WAIT_PRODUCER_EMPTY)) break;
                mbar_expect_tx(smem_u32(&bar_act_full[as]), (uint32_t)n_inst * 256u); // two blocks of n_inst rows x 128 bytes
                tma_load_3d(act_ring + as * C::ACT_BYTES, &tmAct, u * UNIT_K, m_base, 0, smem_u32(&bar_act_full[as]));
                tma_load_3d(act_ring + as * C::ACT_BYTES + C::ACT_HALF, &tmAct, u * UNIT_K + BKE, m_base, 0, smem_u32(&bar_act_full[as]));
                if (++as == ACT_STAGES) { as = 0; aphase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp walks the loop and keeps addresses and descriptors warp-uniform; one elected lane issues.
        // UMMA N = the activation rows of this pass rounded up to 16.
        const uint32_t idesc = make_idesc(0u /*F16*/, false, false, BW, (uint32_t)n_inst);
        const uint64_t desc0 = make_smem_desc_sw128(act_ring, 16, 1024);
        int ws = 0;
        uint32_t wphase = 0;
        bool ok = true;
        for (int i = 0; i < n_units; ++i) {
            // One wait per unit: the first dequantising warp of the unit's group has seen the unit's activations
            // arrive before it reports its rows (below), so this barrier covers both operands.
            ok = mbar_wait_short_warp(smem_u32(&bar_w_full[ws]), wphase, &abort_flag, p.status, WAIT_MMA_FULL);
            if (!ok) break;
            tc_fence_after();
            const uint32_t w0 = tmem_base + (uint32_t)(MB + ws * W_COLS);
            const uint64_t d0 = desc0 + (uint64_t)((uint32_t)(ws * C::ACT_BYTES) >> 4); // the start-address field counts 16 bytes
            if (elect_one()) {
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)
                    umma_a_tmem(tmem_base, w0 + (uint32_t)(ks * 8), d0 + (uint64_t)(((ks >> 2) * C::ACT_HALF + (ks & 3) * 32) >> 4), idesc,
                                (i | ks) ? 1u : 0u);
                umma_commit(smem_u32(&bar_w_empty[ws])); // the unit in tensor memory and its activations are free
            }
            __syncwarp();
            if (++ws == W_STAGES) { ws = 0; wphase ^= 1u; }
        }
        if (ok && elect_one()) umma_commit(smem_u32(&bar_acc_full));
        __syncwarp();
    } else {
        // ------------------------------------------------------------ dequantise (warps 3..10)
        // Thread = weight row; warps 3..6 take the even units of the CTA's walk, warps 7..10 the odd ones, each
        // unit whole (128 k = 64 columns of the row's tensor-memory lane), so that a warp passes one set of
        // hand-offs (weight ring, operand stage, store fence) per 128 k instead of per 64.
        // A thread's row is the tensor-memory lane its warp may write: quadrant warp % 4.
        const int dq = threadIdx.x - DQ_FIRST; // 0..255
        const int grp = (warp - 3) >> 2, row = (warp & 3) * 32 + lane;
        // The prefetched scales go to shared memory; the eight warps meet on a named barrier of their own.
        if (!BTM_I4TC_SCALES_DIRECT) {
#pragma unroll
            for (int j = 0; j < SC_PRE; ++j) {
                const int i = dq + j * 256;
                if (i < sc_total) sc_s[i] = sc_pre[j];
            }
            for (int i = dq + SC_PRE * 256; i < sc_total; i += 256) {
                const int r = i / g_cnt, g = i - r * g_cnt;
                sc_s[i] = __ldg(scales + (size_t)min(n0 + r, p.N - 1) * G + g_first + g);
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
        }
        const __half *srow = sc_s + row * g_cnt - g_first;
        const __half *grow = scales + (size_t)min(n0 + row, p.N - 1) * G;
        const uint32_t xs = (uint32_t)((row >> 1) & 3);
        const uint32_t raw_row0 = raw_ring + (uint32_t)row * 64u;
        const uint32_t tmem_row = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)MB;
        bool ok = true;
        for (int i = grp; ok && i < n_units; i += 2) {
            const int u = unit_at(i);
            const int rs = i % RAW_STAGES, ws = i % W_STAGES;
            ok = mbar_wait_short_warp(smem_u32(&bar_raw_full[rs]), (uint32_t)((i / RAW_STAGES) & 1), &abort_flag, p.status, WAIT_EPI_STAGE);
            if (!ok) break;
            uint4 pw[4]; // 64 packed bytes = 128 nibbles of this row, k = u*128 .. +128
#pragma unroll
            for (int c = 0; c < 4; ++c)
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(pw[c].x), "=r"(pw[c].y), "=r"(pw[c].z), "=r"(pw[c].w)
                             : "r"(raw_row0 + rs * RAW_BYTES + ((((uint32_t)c) ^ xs) << 4)));
            __half2 s0, s1;
            if (BTM_I4TC_SCALES_DIRECT) {
                s0 = __half2half2(sd0);
                s1 = __half2half2(sd1);
                if (i + 2 < n_units) { // the scales of this warp group's next unit, in flight while this one is unpacked
                    const int un = unit_at(i + 2);
                    sd0 = __ldg(grow + (un * UNIT_K) / group);
                    sd1 = __ldg(grow + (un * UNIT_K + BKE) / group);
                }
            } else {
                s0 = __half2half2(srow[(u * UNIT_K) / group]);
                s1 = __half2half2(srow[(u * UNIT_K + BKE) / group]);
            }
            uint4 d[8];
            d[0] = dequant_word(pw[0].x, s0);
            d[1] = dequant_word(pw[0].y, s0);
            d[2] = dequant_word(pw[0].z, s0);
            d[3] = dequant_word(pw[0].w, s0);
            d[4] = dequant_word(pw[1].x, s0);
            d[5] = dequant_word(pw[1].y, s0);
            d[6] = dequant_word(pw[1].z, s0);
            d[7] = dequant_word(pw[1].w, s0);
            ok = mbar_wait_short_warp(smem_u32(&bar_w_empty[ws]), (uint32_t)((i / W_STAGES) & 1) ^ 1u, &abort_flag, p.status, WAIT_EPI_STAGE);
            if (!ok) break;
            tc_fence_after(); // the MMAs that read this stage have completed (their commit released it)
            // 64 fp16 of this row = 32 columns of its tensor-memory lane, two consecutive k per column
            tmem_st_32x32(tmem_row + (uint32_t)(ws * W_COLS), *reinterpret_cast<const uint32_t(*)[32]>(&d[0]));
            d[0] = dequant_word(pw[2].x, s1);
            d[1] = dequant_word(pw[2].y, s1);
            d[2] = dequant_word(pw[2].z, s1);
            d[3] = dequant_word(pw[2].w, s1);
            d[4] = dequant_word(pw[3].x, s1);
            d[5] = dequant_word(pw[3].y, s1);
            d[6] = dequant_word(pw[3].z, s1);
            d[7] = dequant_word(pw[3].w, s1);
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_raw_empty[rs])); // this warp's rows of the unit are in registers
            tmem_st_32x32(tmem_row + (uint32_t)(ws * W_COLS + 32), *reinterpret_cast<const uint32_t(*)[32]>(&d[0]));
            tmem_st_wait();
            tc_fence_before();
            // The activations of the unit come from L2 and have been there for a while; the warp that vouches for
            // them takes this off the MMA issuer's serial path.
            if ((warp & 3) == 3) {
                ok = mbar_wait_short_warp(smem_u32(&bar_act_full[ws]), (uint32_t)((i / W_STAGES) & 1), &abort_flag, p.status, WAIT_EPI_STAGE);
                if (!ok) break;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_w_full[ws]));
        }
        if (ok) mbar_wait_short_warp(smem_u32(&bar_acc_full), 0u, &abort_flag, p.status, WAIT_EPI_TMEM_FULL); // short polls: the wake-up of a long sleep is on the critical path here
        tc_fence_after();
    }

    // ---------------------------------------------------------------- split-K reduction and output
    // Every thread of every CTA of the cluster passes the same two cluster barriers, whatever happened above.
    __syncthreads(); // this CTA's rings are dead: its tensor-core and TMA traffic is over
    const bool acc_ok = abort_flag == 0; // the same answer in every thread of the CTA
    const bool epi = warp >= 3;
    // Every CTA parks its accumulator in its own shared memory ([column = activation row][128 weight rows] fp32, a
    // warp writes 128 contiguous bytes); after one cluster barrier CTA r sums block r of the columns over all CTAs
    // of the cluster (always in rank order, so the sum does not depend on who adds or when) and stores those rows
    // of the output. Nothing is written into another CTA's memory, and the reduction, the conversion and the
    // stores are spread over the cluster instead of queued in its first CTA.
    const int valid = min(MB, p.M - m_base); // columns that hold rows of the activations; the rest is padding
    float *park = reinterpret_cast<float *>(smem_al);
    if (epi) {
        const int quad = warp & 3, erow = quad * 32 + lane; // the tensor-memory lanes this warp may read
#pragma unroll 1
        for (int col0 = ((warp - 3) >> 2) * 32; col0 < valid; col0 += 64) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)col0, v);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) park[(col0 + c) * BW + erow] = __uint_as_float(v[c]);
        }
    }
    cluster_sync_all(); // every accumulator of the cluster is parked and visible (release / acquire)
    if (epi) asm volatile("griddepcontrol.wait;" ::: "memory"); // long since true; orders this grid's stores behind the predecessor
    const int t = threadIdx.x - DQ_FIRST;
    const int per = (((valid + 7) >> 3) + (int)csize - 1) / (int)csize * 8; // columns per CTA, a multiple of 8
    const int c_lo = min(valid, (int)crank * per), c_hi = min(valid, c_lo + per);
    uint16_t *tile_out = reinterpret_cast<uint16_t *>(smem_al + MB * BW * 4); // fp16 [column][128 n] behind the parked values
    if (epi && acc_ok) {
        // A thread sums four consecutive weight rows of every eighth column: 16-byte loads, a warp reads one whole
        // parked column (512 bytes) per load, and all loads of a batch are in flight before the first sum.
        const int r4 = (t & 31) * 4, cw = t >> 5;
        uint32_t src[MAX_SPLIT];
#pragma unroll
        for (int r = 0; r < MAX_SPLIT; ++r) src[r] = map_to_cta(smem_base + (uint32_t)r4 * 4u, (uint32_t)(r < (int)csize ? r : 0));
        constexpr int CB = 4;
#pragma unroll 1
        for (int c0 = c_lo + cw; c0 < c_hi; c0 += 8 * CB) {
            float4 x[CB][MAX_SPLIT];
#pragma unroll
            for (int j = 0; j < CB; ++j) {
                const uint32_t off = (uint32_t)(c0 + 8 * j) * (BW * 4);
#pragma unroll
                for (int r = 0; r < MAX_SPLIT; ++r)
                    if (c0 + 8 * j < c_hi && r < (int)csize)
                        asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                     : "=f"(x[j][r].x), "=f"(x[j][r].y), "=f"(x[j][r].z), "=f"(x[j][r].w)
                                     : "r"(src[r] + off));
            }
#pragma unroll
            for (int j = 0; j < CB; ++j) {
                if (c0 + 8 * j < c_hi) {
                    float4 acc = x[j][0]; // rank order: the sum does not depend on who adds or when
#pragma unroll
                    for (int r = 1; r < MAX_SPLIT; ++r)
                        if (r < (int)csize) {
                            acc.x += x[j][r].x;
                            acc.y += x[j][r].y;
                            acc.z += x[j][r].z;
                            acc.w += x[j][r].w;
                        }
                    const __half2 h01 = __floats2half2_rn(acc.x, acc.y), h23 = __floats2half2_rn(acc.z, acc.w);
                    *reinterpret_cast<uint2 *>(tile_out + (c0 + 8 * j - c_lo) * BW + r4) =
                        make_uint2(*reinterpret_cast<const uint32_t *>(&h01), *reinterpret_cast<const uint32_t *>(&h23));
                }
            }
        }
    }
    // This thread has read what it needs of the other CTAs' shared memory: tell them now and wait for them at the
    // very end, so that the conversion barrier and the global stores do not sit in front of anybody's exit.
    // (relaxed: the arrival publishes nothing, it only says that this thread's loads have returned, which they
    // have, their values having been summed.)
    asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory");
    if (epi && acc_ok) {
        uint16_t *out = reinterpret_cast<uint16_t *>(p.C[0]);
        const bool vec_store = (p.ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        // rows of 256 contiguous bytes to global memory
        const int chunk = t & 15, n = n0 + chunk * 8;
        for (int mt = t >> 4; mt < c_hi - c_lo; mt += 16) {
            const int m = m_base + c_lo + mt;
            if (n < p.N) {
                const uint4 val = *reinterpret_cast<const uint4 *>(tile_out + mt * BW + chunk * 8);
                uint16_t *dst = out + (long long)m * p.ldc + n;
                if (vec_store && n + 8 <= p.N) {
                    *reinterpret_cast<uint4 *>(dst) = val;
                } else {
                    const uint32_t w[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        if (n + e < p.N) dst[e] = (uint16_t)((e & 1) ? (w[e >> 1] >> 16) : (w[e >> 1] & 0xFFFFu));
                }
            }
        }
    }
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); // every CTA has read what it needs of this one's parked accumulator

    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, TMEM_COLS);
    }
}

int configure_int4_tc_kernels()
{
    using namespace i4tc;
    cudaError_t e = cudaFuncSetAttribute(int4_gemm_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<64>::SMEM_BYTES + SCALE_SMEM_MAX);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(int4_gemm_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<128>::SMEM_BYTES + SCALE_SMEM_MAX);
    return check_cuda(e, "cudaFuncSetAttribute(int4_gemm_tc)");
}

// Preconditions (checked by the caller): K % 128 == 0, group % 64 == 0, K % group == 0, act / w / out
// 16-byte aligned, M > 0. Returns BTM_ERR_UNSUPPORTED (nothing launched) when the scales of one K slice do
// not fit the shared memory set aside for them; the caller then takes the general kernel.
int launch_int4_gemm_tc(cudaStream_t st, int M, int N, int K, int group, const void *act, const void *w, const void *scales, void *out,
                        int *status, int sm_count)
{
    using namespace i4tc;
    const int units = K / UNIT_K;
    const int tiles = (N + BW - 1) / BW;
    // K split: as many CTAs per weight tile as the machine holds at two CTAs per SM.
    int split = (2 * sm_count) / tiles;
    split = split < 1 ? 1 : split > MAX_SPLIT ? MAX_SPLIT : split;
    if (split > units) split = units;
    const int groups_per_slice = ((units + split - 1) / split * UNIT_K + group - 1) / group + 1;
    const size_t sc_bytes = (size_t)BW * groups_per_slice * 2;
    if (sc_bytes > SCALE_SMEM_MAX) return BTM_ERR_UNSUPPORTED;
    CUtensorMap tmAct, tmW;
    int rc = encode_tmap_3d(&tmW, BTM_U8, w, (uint64_t)K / 2, (uint64_t)N, 1, (uint64_t)K / 2, (uint64_t)K / 2, 64, BW, 2 /*64-byte swizzle*/);
    if (rc) return rc;
    for (int m_base = 0; m_base < M; m_base += 128) {
        const int rows = M - m_base < 128 ? M - m_base : 128;
        const int mb = rows <= 64 ? 64 : 128;
        const int n_inst = (rows + 15) / 16 * 16; // rows the activation tiles carry and the MMAs multiply
        rc = encode_tmap_3d(&tmAct, BTM_F16, act, (uint64_t)K, (uint64_t)M, 1, (uint64_t)K * 2, (uint64_t)K * 2, 64, (uint32_t)n_inst);
        if (rc) return rc;
        GemmParams p;
        memset(&p, 0, sizeof(p));
        p.M = M;
        p.N = N;
        p.K = K;
        p.batch = 1;
        p.ndst = 1;
        p.C[0] = out;
        p.ldc = N;
        p.status = status;
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3((unsigned)(tiles * split), 1, 1);
        cfg.blockDim = dim3(THREADS, 1, 1);
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)split;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization; // the kernel orders itself with griddepcontrol
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        cudaError_t e;
        if (mb == 64) {
            cfg.dynamicSmemBytes = Cfg<64>::SMEM_BYTES + sc_bytes;
            e = cudaLaunchKernelEx(&cfg, int4_gemm_tc_kernel<64>, tmAct, tmW, p, (const __half *)scales, group, m_base, n_inst);
        } else {
            cfg.dynamicSmemBytes = Cfg<128>::SMEM_BYTES + sc_bytes;
            e = cudaLaunchKernelEx(&cfg, int4_gemm_tc_kernel<128>, tmAct, tmW, p, (const __half *)scales, group, m_base, n_inst);
        }
        rc = check_cuda(e, "int4 tensor-core matmul launch");
        if (rc) return rc;
    }
    return BTM_OK;
}

} // namespace btm
