// Two-SM tensor-core matmul for sm_100a (16-bit inputs): the same product as gemm_tc.cu, with the
// tile of a CTA PAIR being 256 x 256. Each CTA of the pair holds 128 rows of A and half of the B
// columns; one tcgen05.mma.cta_group::2 issued by the leader CTA drives both SMs' tensor cores, each
// reading B from both CTAs' shared memory. Per 128x256x64 block of work a CTA therefore fetches
// 32 KB (16 KB of A + 16 KB of B) instead of 48 KB, which is what the one-CTA kernel is limited by
// (L2 -> SM traffic). No cluster-multicast load is used: every CTA issues plain TMA loads for its own
// halves and only the mbarrier completion targets the leader (cp.async.bulk.tensor ... cta_group::2).
//
// Tile list = full tiles, then half-width (256 x 128) tiles for what would otherwise be a partly
// filled last wave: T tiles on C clusters with r = T mod C and 2r <= C run the last r tiles as 2r half
// tiles, which shortens the tail from one tile time to half of one.
//
// Roles per CTA (192 threads): warp 0 TMA producer, warp 1 tensor-memory owner (+ MMA issue in the
// leader), warps 2-5 epilogue for this CTA's 128 rows. Barriers: full[s] lives in the leader and
// counts the bytes of both CTAs; empty[s] and tmem_full[a] exist in both CTAs and are signalled by
// multicast tcgen05.commit; tmem_empty[a] lives in the leader and collects the 8 epilogue warps.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "btm_internal.h"
#include "btm_ptx.cuh"
#include "gemm_epilogue.cuh"

namespace btm {

namespace tc2 {
constexpr int PAIR_M = 256;       // rows of a pair tile
constexpr int CTA_M = 128;        // rows per CTA = accumulator lanes
constexpr int BN = 256;           // full tile width
constexpr int BKE = 64;           // k elements per stage (128 bytes)
constexpr int A_BYTES = CTA_M * 128;
constexpr int CHUNK_BYTES = BKE * 128; // one 64-column B chunk: 64 k-rows x 128 B
constexpr int KB_BYTES = A_BYTES + 2 * CHUNK_BYTES; // one 64-deep k-block of a CTA: 16 KB of A + 16 KB of B
// k-blocks per pipeline stage: a stage is handed over (one full / empty barrier round trip, one commit) per KPS
// k-blocks, i.e. per 4 * KPS tcgen05.mma. Measured at fp16 4096^3 under the power cap, same run as the library's
// kernel on the same buffers: KPS 1 (six stages of 32 KB) 1076 TFLOP/s = 0.89 of the library, KPS 2 (three stages of
// 64 KB) 1132 = 0.95, KPS 3 (two stages of 96 KB) 1047 = 0.875.
#ifndef BTM_TC2_KPS
#define BTM_TC2_KPS 2
#endif
constexpr int KPS = BTM_TC2_KPS;
constexpr int STAGE_BYTES = KPS * KB_BYTES;
#ifndef BTM_TC2_STAGES
#define BTM_TC2_STAGES (6 / BTM_TC2_KPS)
#endif
constexpr int STAGES = BTM_TC2_STAGES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_SMEM_BYTES + 1024; // ring + epilogue staging + alignment slack
constexpr int TMEM_COLS = 512;    // two 256-column accumulators
constexpr int THREADS = 192;
} // namespace tc2

struct PairTile {
    int b, m, n0, bn; // product, pair-row index, first column, width (256 or 128)
};

__device__ __forceinline__ PairTile decode_pair_tile(const GemmParams &p, int t)
{
    int big = t, half = -1;
    if (t >= p.tiles_full) {
        const int s = t - p.tiles_full;
        big = p.tiles_full + (s >> 1);
        half = s & 1;
    }
    const int per_batch = p.tiles_m * p.tiles_n;
    PairTile o;
    o.b = big / per_batch;
    const int r0 = big - o.b * per_batch;
    const int per_group = p.group_m * p.tiles_n;
    const int gid = r0 / per_group;
    const int first_m = gid * p.group_m;
    const int gsz = min(p.tiles_m - first_m, p.group_m);
    const int r = r0 - gid * per_group;
    o.m = first_m + r % gsz;
    const int n = r / gsz;
    o.bn = half < 0 ? tc2::BN : tc2::BN / 2;
    o.n0 = n * tc2::BN + (half > 0 ? tc2::BN / 2 : 0);
    return o;
}

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t cta)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta));
    return r;
}

template <int DT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(tc2::THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ StoreMaps cmaps, const GemmParams p)
{
    using namespace tc2;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[STAGES];     // used in the leader: bytes of both CTAs
    __shared__ __align__(8) uint64_t bar_empty[STAGES];    // per CTA, signalled by multicast commit
    __shared__ __align__(8) uint64_t bar_tmem_full[2];     // per CTA, signalled by multicast commit
    __shared__ __align__(8) uint64_t bar_tmem_empty[2];    // used in the leader: 8 epilogue warps
    __shared__ uint32_t tmem_base_holder;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank(); // 0 = leader
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int total_tiles = p.tiles_full + p.tiles_tail;

    // Programmatic dependent launch: a product that follows this one on the stream may become resident wherever an
    // SM pair falls free and set itself up; it reads its operands (and so writes its output) only after this grid
    // has completed (griddepcontrol.wait in its producers).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bar_tmem_full[a]), 1);
            mbar_init(smem_u32(&bar_tmem_empty[a]), 8);
        }
        fence_mbar_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    if (warp == 1) {
        tmem_alloc<2>(smem_u32(&tmem_base_holder), TMEM_COLS);
        tmem_relinquish<2>();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all(); // the peer's barriers exist before anything remote can reach them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_holder;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0 && !p.debug_skip_loads) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // The operands may be the predecessor's output. Every other role, the stores of C included, depends on
            // these loads through the stage barriers.
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int tile = cluster_id; ok && tile < total_tiles; tile += num_clusters) {
                const PairTile pt = decode_pair_tile(p, tile);
                const int half_bn = pt.bn >> 1;      // columns of B this CTA loads
                const int chunks = half_bn >> 6;     // 64-column chunks: 2 or 1
                const uint32_t cta_bytes = (uint32_t)(A_BYTES + chunks * CHUNK_BYTES);
                for (int kb = 0; kb < p.num_kb; kb += KPS) {
                    if (!mbar_wait<true>(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag, p.status, WAIT_PRODUCER_EMPTY, p.wait_limit)) {
                        ok = false;
                        break;
                    }
                    const int nsub = min(KPS, p.num_kb - kb); // k-blocks in this stage (the last stage of a tile may be short)
                    const uint32_t full_local = smem_u32(&bar_full[stage]);
                    if (rank == 0) mbar_expect_tx(full_local, 2u * cta_bytes * (uint32_t)nsub);
                    const uint32_t full_leader = map_to_cta(full_local, 0);
                    for (int sub = 0; sub < nsub; ++sub) {
                        const uint32_t sbase = smem_base + stage * STAGE_BYTES + sub * KB_BYTES;
                        const int k0 = (kb + sub) * BKE;
                        tma_load_3d_2sm(sbase, &tmA, k0, pt.m * PAIR_M + (int)rank * CTA_M, pt.b, full_leader);
                        for (int c = 0; c < chunks; ++c)
                            tma_load_3d_2sm(sbase + A_BYTES + c * CHUNK_BYTES, &tmB, pt.n0 + (int)rank * half_bn + c * 64, k0, pt.b, full_leader);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t fmt = DT == BTM_BF16 ? 1u : 0u;
            constexpr uint32_t idesc_full = make_idesc(fmt, false, true, PAIR_M, BN);
            constexpr uint32_t idesc_half = make_idesc(fmt, false, true, PAIR_M, BN / 2);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = cluster_id; ok && tile < total_tiles; tile += num_clusters, ++it) {
                const PairTile pt = decode_pair_tile(p, tile);
                const uint32_t idesc = pt.bn == BN ? idesc_full : idesc_half;
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait<true>(smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1u, &abort_flag, p.status, WAIT_MMA_TMEM_EMPTY, p.wait_limit)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < p.num_kb; kb += KPS) {
                    if (!mbar_wait<true>(smem_u32(&bar_full[stage]), phase, &abort_flag, p.status, WAIT_MMA_FULL, p.wait_limit)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const int nsub = min(KPS, p.num_kb - kb);
                    // One descriptor pair per stage; a k-block or k-step only moves the start-address field (which
                    // counts 16 bytes), so every further descriptor is one addition.
                    const uint64_t ad0 = make_smem_desc_sw128(smem_base + stage * STAGE_BYTES, 16, 1024);
                    const uint64_t bd0 = make_smem_desc_sw128(smem_base + stage * STAGE_BYTES + A_BYTES, CHUNK_BYTES, 1024);
                    for (int sub = 0; sub < nsub; ++sub) {
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            const uint64_t ad = ad0 + (uint64_t)((sub * KB_BYTES + ks * 32) >> 4);
                            const uint64_t bd = bd0 + (uint64_t)((sub * KB_BYTES + ks * 16 * 128) >> 4);
                            umma<2, false>(d_tmem, ad, bd, idesc, (uint32_t)((kb | sub | ks) != 0));
                        }
                    }
                    umma_commit_2sm(smem_u32(&bar_empty[stage]), (uint16_t)3);
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) umma_commit_2sm(smem_u32(&bar_tmem_full[acc]), (uint16_t)3);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        const int quad = warp & 3;
        const uint32_t epi_smem = smem_base + STAGES * STAGE_BYTES + (uint32_t)quad * EPI_WARP_BYTES;
        uint32_t epi_tiles = 0;
        int it = 0;
        for (int tile = cluster_id; tile < total_tiles; tile += num_clusters, ++it) {
            const PairTile pt = decode_pair_tile(p, tile);
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            // One lane waits and broadcasts the outcome: tcgen05.ld below needs the whole warp.
            if (!mbar_wait_warp<true>(smem_u32(&bar_tmem_full[acc]), acc_phase, &abort_flag, p.status, WAIT_EPI_TMEM_FULL, p.wait_limit)) break;
            tc_fence_after();
            epilogue_band<DT>(p, cmaps, tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN),
                              pt.m * PAIR_M + (int)rank * CTA_M + quad * 32, pt.n0, pt.bn, pt.b, epi_smem, epi_tiles, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(smem_u32(&bar_tmem_empty[acc]));
                else mbar_arrive_cluster(smem_u32(&bar_tmem_empty[acc]), 0);
            }
        }
        epilogue_drain(lane);
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
        __syncthreads();
    }
    cluster_sync_all(); // neither CTA leaves while the other may still touch its shared memory
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc<2>(tmem_base, TMEM_COLS);
    }
}

template <int DT>
static int launch_pair(cudaStream_t st, int sm_count, const CUtensorMap &tmA, const CUtensorMap &tmB, const StoreMaps &cm, GemmParams p)
{
    using namespace tc2;
    p.tiles_m = (p.M + PAIR_M - 1) / PAIR_M;
    p.tiles_n = (p.N + BN - 1) / BN;
    p.num_kb = (p.K + BKE - 1) / BKE;
    if (p.group_m <= 0) p.group_m = 8; // measured against 4, 6, 12, 16 on 16384^3, its column shards and 4096^3
    const long long total = (long long)p.batch * p.tiles_m * p.tiles_n;
    if (total <= 0) return BTM_OK;
    if (total > 0x3FFFFFFFLL) return set_error(BTM_ERR_UNSUPPORTED, "too many output tiles (%lld)", total);
    // How many CTA pairs the device can hold at once (GPC boundaries can make it less than SMs/2).
    static int resident_pairs[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && resident_pairs[dev] == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(sm_count & ~1);
        cfg.blockDim = dim3(THREADS);
        cfg.dynamicSmemBytes = SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel<DT>, &cfg) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = sm_count / 2;
        }
        resident_pairs[dev] = n < sm_count / 2 ? n : sm_count / 2;
        if (getenv("BTM_DEBUG")) fprintf(stderr, "[btm] device %d holds %d CTA pairs of the two-SM kernel at once\n", dev, n);
    }
    const int max_clusters = (dev >= 0 && dev < 64) ? resident_pairs[dev] : sm_count / 2;
    const int rem = (int)(total % max_clusters);
    int tail_big = 0;
    if (rem > 0 && 2 * rem <= max_clusters) tail_big = rem; // run the last `rem` tiles as 2*rem half-width tiles
    p.tiles_full = (int)total - tail_big;
    p.tiles_tail = 2 * tail_big;
    const long long sched = (long long)p.tiles_full + p.tiles_tail;
    const int clusters = (int)(sched < max_clusters ? sched : max_clusters);
    cudaLaunchConfig_t lc;
    memset(&lc, 0, sizeof(lc));
    lc.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
    lc.blockDim = dim3(THREADS, 1, 1);
    lc.dynamicSmemBytes = SMEM_BYTES;
    lc.stream = st;
    cudaLaunchAttribute pdl;
    pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization; // the kernel orders itself with griddepcontrol
    pdl.val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = &pdl;
    lc.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&lc, gemm_tc2_kernel<DT>, tmA, tmB, cm, p), "gemm_tc2 launch");
}

int configure_gemm_tc2_kernels()
{
    cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel<BTM_F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc2::SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc2_kernel<BTM_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, tc2::SMEM_BYTES);
    return check_cuda(e, "cudaFuncSetAttribute(gemm_tc2)");
}

int launch_gemm_tc2(int dtype, cudaStream_t st, int sm_count, const CUtensorMap &tmA, const CUtensorMap &tmB, const StoreMaps &cm,
                    const GemmParams &p)
{
    if (dtype == BTM_F16) return launch_pair<BTM_F16>(st, sm_count, tmA, tmB, cm, p);
    if (dtype == BTM_BF16) return launch_pair<BTM_BF16>(st, sm_count, tmA, tmB, cm, p);
    return set_error(BTM_ERR_UNSUPPORTED, "two-SM matmul: dtype %d is not supported", dtype);
}

} // namespace btm
