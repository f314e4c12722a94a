// Tensor-core matmul for sm_100a: C[M,N] = A[M,K] . B[K,N], row-major, fp32 accumulation.
//
// One persistent CTA per SM walks a static list of 128 x BN output tiles (all products of a
// batched call share one list). Inside a CTA the work is split by warp:
//   warp 0      TMA producer: streams 128-byte-wide k-slices of A and B into a ring of
//               shared-memory stages (128-byte swizzle), one mbarrier per stage;
//   warp 1      owns tensor memory and issues tcgen05.mma (one elected lane); accumulators
//               live in tensor memory, two of them, so the epilogue of tile i overlaps the
//               main loop of tile i+1;
//   warps 2-5   epilogue: tcgen05.ld the accumulator (one 32-row quadrant per warp), round to
//               the output type and store to C — to every destination when the call carries
//               peer copies of C (the fused all-gather of the N-sharded product).
// A is K-major in shared memory. B is row-major [K,N] in global memory, so it is loaded as
// N-contiguous 128-byte chunks and consumed as an MN-major operand; no transpose pass exists.
// fp32 inputs run as a three-term TF32 split: z = 0/1 of the tensor maps select the hi and lo
// planes prepared by split_tf32_kernel and each k-step issues hi.hi, hi.lo and lo.hi.
#include <cstring>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "btm_internal.h"
#include "btm_ptx.cuh"
#include "gemm_epilogue.cuh"

namespace btm {

constexpr int BM = 128;          // rows of one output tile = accumulator lanes
constexpr int SLICE_BYTES = 128; // bytes of K (for A) or N (for B) per shared-memory row = swizzle span
constexpr int UMMA_K_BYTES = 32; // bytes of K consumed by one tcgen05.mma
constexpr int NUM_THREADS = 192;
#ifndef BTM_TC1_KPS
#define BTM_TC1_KPS 1
#endif

template <int BN, int DT, bool BT = false, bool AT = false>
struct TileCfg {
    static constexpr bool kTf32 = (DT == BTM_F32);
    static constexpr int kEs = kTf32 ? 4 : 2;              // element bytes
    static constexpr int kBKE = SLICE_BYTES / kEs;          // k elements per stage
    static constexpr int kPlanes = kTf32 ? 2 : 1;           // hi/lo planes
    // 16-bit B stays row-major [K,N] in global memory and is consumed MN-major: BN/64 chunks of
    // kBKE rows x 128 B. The fp32 planes are written transposed ([N,K]) by the split pass, so B
    // is K-major like A: BN rows x 128 B from a single TMA box.
    static constexpr bool kBMnMajor = !kTf32 && !BT; // BT: the caller's B is already [N,K] (K-major)
    // AT: the caller's A is stored [K,M] (M contiguous): it is loaded as M-contiguous 128-byte chunks (BM/64 of them,
    // 64 k-rows x 128 B each) and consumed as an MN-major operand, exactly as B is when it is row-major [K,N].
    static constexpr bool kAMnMajor = !kTf32 && AT;
    static constexpr int kAChunks = BM / (SLICE_BYTES / kEs);
    static constexpr int kChunkN = SLICE_BYTES / kEs;       // n elements per MN-major B chunk
    static constexpr int kChunks = BN / kChunkN;            // MN-major B chunks per stage
    static constexpr int kChunkBytes = kBKE * SLICE_BYTES;  // one MN-major chunk: kBKE rows of 128 B
    static constexpr int kABytes = BM * SLICE_BYTES;        // one A plane
    static constexpr int kBBytes = BN * SLICE_BYTES;        // one B plane (either major)
    static constexpr int kKbBytes = kPlanes * (kABytes + kBBytes); // one k-block of operands
    // k-blocks per pipeline stage (16-bit kernels; the fp32 planes leave no room): one barrier round trip and one
    // commit per kKps k-blocks, as in the two-SM kernel.
    static constexpr int kKps = kTf32 ? 1 : BTM_TC1_KPS;
    static constexpr int kStageBytes = kKps * kKbBytes;
    static constexpr int kStages = (kKbBytes <= 48 * 1024 ? 4 : 3) / kKps;
    static constexpr int kSmemBytes = kStages * kStageBytes + EPI_SMEM_BYTES + 1024; // ring + epilogue staging + alignment slack
    static constexpr int kTmemCols = 2 * BN;                // two accumulators
    static constexpr int kKSteps = SLICE_BYTES / UMMA_K_BYTES;
    static constexpr int kUmmaKRows = UMMA_K_BYTES / kEs;   // k rows of B per mma
    static_assert(kTmemCols == 128 || kTmemCols == 256 || kTmemCols == 512, "tensor memory columns must be a power of two");
};

struct TileCoord {
    int b, m, n0, bn; // product, row-tile index, first column, width (BN, or BN/2 for a tail tile)
};

// The tile list is `tiles_full` full-width tiles followed by `tiles_tail` half-width ones: the tiles
// of a partly filled last wave are run as twice as many half tiles, which halves the tail.
template <int BN>
__device__ __forceinline__ TileCoord decode_tile(const GemmParams &p, int tile_in_list)
{
    int tile = tile_in_list, half = -1;
    if (tile_in_list >= p.tiles_full) {
        const int s = tile_in_list - p.tiles_full;
        tile = p.tiles_full + (s >> 1);
        half = s & 1;
    }
    const int per_batch = p.tiles_m * p.tiles_n;
    TileCoord c;
    c.b = tile / per_batch;
    const int t = tile - c.b * per_batch;
    const int per_group = p.group_m * p.tiles_n;
    const int gid = t / per_group;
    const int first_m = gid * p.group_m;
    const int gsz = min(p.tiles_m - first_m, p.group_m);
    const int r = t - gid * per_group;
    c.m = first_m + r % gsz;
    c.bn = half < 0 ? BN : BN / 2;
    c.n0 = (r / gsz) * BN + (half > 0 ? BN / 2 : 0);
    return c;
}

template <int BN, int DT, bool BT = false, bool AT = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ StoreMaps cmaps, const GemmParams p)
{
    using Cfg = TileCfg<BN, DT, BT, AT>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[Cfg::kStages];
    __shared__ __align__(8) uint64_t bar_empty[Cfg::kStages];
    __shared__ __align__(8) uint64_t bar_tmem_full[2];
    __shared__ __align__(8) uint64_t bar_tmem_empty[2];
    __shared__ uint32_t tmem_base_holder;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u; // swizzle atoms need 1024-byte alignment
    const int total_tiles = p.tiles_full + p.tiles_tail;

    // Programmatic dependent launch: a product that follows this one on the stream may become resident wherever an
    // SM falls free and set itself up; it reads its operands (and so writes its output) only after this grid has
    // completed (griddepcontrol.wait in its producer).
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bar_tmem_full[a]), 1);
            mbar_init(smem_u32(&bar_tmem_empty[a]), 4); // one arrival per epilogue warp
        }
        fence_mbar_init();
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(&tmem_base_holder), Cfg::kTmemCols);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_holder;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0 && !p.debug_skip_loads) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // The product is launched with programmatic stream serialisation: everything up to here (barriers,
            // tensor memory, descriptor prefetch) may have run under its predecessor (for fp32, the pass that writes
            // the operand planes); the operands are read only now. Every other role, the stores of C included,
            // depends on these loads through the stage barriers.
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const TileCoord tc = decode_tile<BN>(p, tile);
                for (int kb = 0; kb < p.num_kb; kb += Cfg::kKps) {
                    if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag, p.status, WAIT_PRODUCER_EMPTY, p.wait_limit)) {
                        ok = false;
                        break;
                    }
                    const int nsub = min(Cfg::kKps, p.num_kb - kb); // the last stage of a tile may be short
                    const uint32_t full = smem_u32(&bar_full[stage]);
                    // A tail tile (16-bit only) loads half of the B chunks.
                    const int chunks = Cfg::kBMnMajor ? tc.bn / Cfg::kChunkN : 0;
                    mbar_expect_tx(full, (uint32_t)nsub * (Cfg::kBMnMajor ? (uint32_t)(Cfg::kABytes + chunks * Cfg::kChunkBytes) : (uint32_t)Cfg::kKbBytes));
                    for (int sub = 0; sub < nsub; ++sub) {
                        const uint32_t sbase = smem_base + stage * Cfg::kStageBytes + sub * Cfg::kKbBytes;
                        const int k0 = (kb + sub) * Cfg::kBKE;
#pragma unroll
                        for (int pl = 0; pl < Cfg::kPlanes; ++pl) {
                            const int z = Cfg::kTf32 ? pl : tc.b;
                            if constexpr (Cfg::kAMnMajor) {
#pragma unroll
                                for (int c = 0; c < Cfg::kAChunks; ++c)
                                    tma_load_3d(sbase + c * Cfg::kChunkBytes, &tmA, tc.m * BM + c * Cfg::kChunkN, k0, z, full);
                            } else {
                                tma_load_3d(sbase + pl * Cfg::kABytes, &tmA, k0, tc.m * BM, z, full);
                            }
                            const uint32_t bbase = sbase + Cfg::kPlanes * Cfg::kABytes + pl * Cfg::kBBytes;
                            if constexpr (Cfg::kBMnMajor) {
#pragma unroll
                                for (int c = 0; c < Cfg::kChunks; ++c)
                                    if (c < chunks) tma_load_3d(bbase + c * Cfg::kChunkBytes, &tmB, tc.n0 + c * Cfg::kChunkN, k0, z, full);
                            } else {
                                tma_load_3d(bbase, &tmB, k0, tc.n0, z, full);
                            }
                        }
                    }
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t kFmt = Cfg::kTf32 ? 2u : (DT == BTM_BF16 ? 1u : 0u);
            constexpr uint32_t idesc_full = make_idesc(kFmt, Cfg::kAMnMajor, Cfg::kBMnMajor, BM, BN);
            constexpr uint32_t idesc_half = make_idesc(kFmt, Cfg::kAMnMajor, Cfg::kBMnMajor, BM, BN / 2);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
                const uint32_t idesc = tile < p.tiles_full ? idesc_full : idesc_half;
                const int acc = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1u, &abort_flag, p.status, WAIT_MMA_TMEM_EMPTY, p.wait_limit)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < p.num_kb; kb += Cfg::kKps) {
                    if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag, p.status, WAIT_MMA_FULL, p.wait_limit)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const int nsub = min(Cfg::kKps, p.num_kb - kb);
                    // One descriptor per operand plane and stage; a k-block or a k-step only moves the start-address
                    // field (it counts 16 bytes), so every further descriptor is one addition instead of a rebuild.
                    // A: K-major, 8-row groups 1024 B apart; a k-step moves 32 B inside the swizzle span.
                    // B: MN-major, n-chunks kChunkBytes apart (leading offset), 8-k-row groups 1024 B
                    // apart (stride offset); a k-step moves kUmmaKRows rows of 128 B.
                    const uint32_t a0 = smem_base + stage * Cfg::kStageBytes, b0 = a0 + Cfg::kPlanes * Cfg::kABytes;
                    const uint64_t a_hi0 = Cfg::kAMnMajor ? make_smem_desc_sw128(a0, Cfg::kChunkBytes, 1024) : make_smem_desc_sw128(a0, 16, 1024);
                    const uint64_t b_hi0 = Cfg::kBMnMajor ? make_smem_desc_sw128(b0, Cfg::kChunkBytes, 1024) : make_smem_desc_sw128(b0, 16, 1024);
                    constexpr uint32_t a_step = (Cfg::kAMnMajor ? Cfg::kUmmaKRows * SLICE_BYTES : UMMA_K_BYTES) >> 4;
                    constexpr uint32_t b_step = (Cfg::kBMnMajor ? Cfg::kUmmaKRows * SLICE_BYTES : UMMA_K_BYTES) >> 4;
                    for (int sub = 0; sub < nsub; ++sub) {
                        const uint32_t sub_off = (uint32_t)(sub * Cfg::kKbBytes) >> 4;
#pragma unroll
                        for (int ks = 0; ks < Cfg::kKSteps; ++ks) {
                            const uint64_t a_hi = a_hi0 + (uint64_t)(sub_off + ks * a_step);
                            const uint64_t b_hi = b_hi0 + (uint64_t)(sub_off + ks * b_step);
                            const uint32_t first = (kb | sub | ks) != 0;
                            if constexpr (Cfg::kTf32) {
                                // the low planes lie kABytes / kBBytes behind the high ones, K-major like them
                                const uint64_t a_lo = a_hi + (uint64_t)(Cfg::kABytes >> 4);
                                const uint64_t b_lo = b_hi + (uint64_t)(Cfg::kBBytes >> 4);
                                umma<1, true>(d_tmem, a_lo, b_hi, idesc, first);
                                umma<1, true>(d_tmem, a_hi, b_lo, idesc, 1u);
                                umma<1, true>(d_tmem, a_hi, b_hi, idesc, 1u);
                            } else {
                                umma<1, false>(d_tmem, a_hi, b_hi, idesc, first);
                            }
                        }
                    }
                    umma_commit(smem_u32(&bar_empty[stage])); // stage reusable once these MMAs have read it
                    if (++stage == Cfg::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) umma_commit(smem_u32(&bar_tmem_full[acc]));
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quad = warp & 3; // tensor-memory lane quadrant this warp may read
        const uint32_t epi_smem = smem_base + Cfg::kStages * Cfg::kStageBytes + (uint32_t)quad * EPI_WARP_BYTES;
        uint32_t epi_tiles = 0;
        int it = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
            const TileCoord tc = decode_tile<BN>(p, tile);
            const int acc = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            // One lane waits and broadcasts the outcome: tcgen05.ld below needs the whole warp.
            if (!mbar_wait_warp(smem_u32(&bar_tmem_full[acc]), acc_phase, &abort_flag, p.status, WAIT_EPI_TMEM_FULL, p.wait_limit)) break;
            tc_fence_after();
            epilogue_band<DT>(p, cmaps, tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN), tc.m * BM + quad * 32, tc.n0,
                              tc.bn, tc.b, epi_smem, epi_tiles, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_tmem_empty[acc]));
        }
        epilogue_drain(lane);
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        // A wait ran out somewhere. Copies already issued by the producer finish on their own
        // within microseconds; give them a bounded grace period before shared memory is released.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {}
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, Cfg::kTmemCols);
    }
}

// Low part of the split. For an infinite x the high part is already x and x - hi would be Inf - Inf = NaN, which
// would turn a whole output row or column into NaN where an fp32 product gives +-Inf; the low part is 0 there.
__device__ __forceinline__ float split_lo(float x, float hi) { return fabsf(x) == INFINITY ? 0.0f : x - hi; }

// 3xTF32 operand preparation: hi = x with the low 13 mantissa bits cleared (what the tensor
// core reads of an fp32 word), lo = x - hi (exact in fp32). Written as two dense planes.
__global__ void split_tf32_kernel(const float *__restrict__ src, long long ld, int rows, int cols,
                                  float *__restrict__ hi, float *__restrict__ lo, long long ld_dst)
{
    const long long total = (long long)rows * ld_dst;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); // the product behind this pass may set itself up now
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / ld_dst;
        const int c = (int)(i - r * ld_dst);
        float x = (c < cols) ? src[r * ld + c] : 0.0f;
        const float h = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
        hi[i] = h;
        lo[i] = split_lo(x, h);
    }
}

// Same split for B, written transposed: src is [rows=K, cols=N] row-major, the planes are
// [N, ld_dst] (K contiguous) so that the tensor cores read B K-major like A.
__global__ void split_tf32_transpose_kernel(const float *__restrict__ src, long long ld, int rows, int cols,
                                            float *__restrict__ hi, float *__restrict__ lo, long long ld_dst)
{
    __shared__ float tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int r = r0 + i, c = c0 + threadIdx.x;
        tile[i][threadIdx.x] = (r < rows && c < cols) ? src[(long long)r * ld + c] : 0.0f;
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int c = c0 + i, r = r0 + threadIdx.x; // output row = source column
        if (c < cols && r < ld_dst) {
            const float x = tile[threadIdx.x][i];
            const float h = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
            hi[(long long)c * ld_dst + r] = h;
            lo[(long long)c * ld_dst + r] = split_lo(x, h);
        }
    }
}

// Both operands in one launch (the 1024^3 product is launch-bound: one kernel less is ~5 us of 30):
// the first `tiles_a` blocks split 32 x 32 tiles of A in place, the others split and transpose tiles of B.
__global__ void split_tf32_pair_kernel(const float *__restrict__ A, long long lda, int M, int K, float *__restrict__ a_hi,
                                       float *__restrict__ a_lo, const float *__restrict__ B, long long ldb, int N,
                                       float *__restrict__ b_hi, float *__restrict__ b_lo, long long Kp, int tiles_a, int kt)
{
    __shared__ float tile[32][33];
    const int blk = blockIdx.x;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); // the product behind this pass may set itself up now
    if (blk < tiles_a) {
        const int r0 = (blk / kt) * 32, c0 = (blk % kt) * 32;
        for (int i = threadIdx.y; i < 32; i += blockDim.y) {
            const int r = r0 + i, c = c0 + threadIdx.x;
            if (r < M && c < Kp) {
                const float x = c < K ? A[(long long)r * lda + c] : 0.0f;
                const float h = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
                a_hi[(long long)r * Kp + c] = h;
                a_lo[(long long)r * Kp + c] = split_lo(x, h);
            }
        }
        return;
    }
    const int b = blk - tiles_a;
    const int c0 = (b / kt) * 32, r0 = (b % kt) * 32; // c0: column of B (output row), r0: row of B = k
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int r = r0 + i, c = c0 + threadIdx.x;
        tile[i][threadIdx.x] = (r < K && c < N) ? B[(long long)r * ldb + c] : 0.0f;
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        const int c = c0 + i, r = r0 + threadIdx.x;
        if (c < N && r < Kp) {
            const float x = tile[threadIdx.x][i];
            const float h = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
            b_hi[(long long)c * Kp + r] = h;
            b_lo[(long long)c * Kp + r] = split_lo(x, h);
        }
    }
}

int launch_split_tf32_pair(cudaStream_t st, const float *A, long long lda, int M, int K, float *a_hi, float *a_lo, const float *B,
                           long long ldb, int N, float *b_hi, float *b_lo, long long Kp)
{
    const long long kt = (Kp + 31) / 32;
    const long long tiles_a = (long long)((M + 31) / 32) * kt, tiles_b = (long long)((N + 31) / 32) * kt;
    if (tiles_a + tiles_b == 0) return BTM_OK;
    if (tiles_a + tiles_b > 0x7FFFFFFFLL) return set_error(BTM_ERR_UNSUPPORTED, "fp32 matmul: operands too large for the split pass");
    split_tf32_pair_kernel<<<(unsigned)(tiles_a + tiles_b), dim3(32, 8), 0, st>>>(A, lda, M, K, a_hi, a_lo, B, ldb, N, b_hi, b_lo, Kp,
                                                                                 (int)tiles_a, (int)kt);
    return check_cuda(cudaGetLastError(), "split_tf32_pair launch");
}

int launch_split_tf32_transpose(cudaStream_t st, const float *src, long long ld, int rows, int cols, float *dst_hi,
                                float *dst_lo, long long ld_dst)
{
    if (rows == 0 || cols == 0) return BTM_OK;
    dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((ld_dst + 31) / 32));
    if (grid.y > 65535) return set_error(BTM_ERR_UNSUPPORTED, "fp32 matmul: K too large for the split pass");
    split_tf32_transpose_kernel<<<grid, dim3(32, 8), 0, st>>>(src, ld, rows, cols, dst_hi, dst_lo, ld_dst);
    return check_cuda(cudaGetLastError(), "split_tf32_transpose launch");
}

int launch_split_tf32(cudaStream_t st, const float *src, long long ld, int rows, int cols, float *dst_hi,
                      float *dst_lo, long long ld_dst)
{
    const long long total = (long long)rows * ld_dst;
    if (total == 0) return BTM_OK;
    const int block = 256;
    const long long want = (total + block - 1) / block;
    const int grid = (int)(want < 148 * 8 ? want : 148 * 8);
    split_tf32_kernel<<<grid, block, 0, st>>>(src, ld, rows, cols, dst_hi, dst_lo, ld_dst);
    return check_cuda(cudaGetLastError(), "split_tf32 launch");
}

template <int BN, int DT, bool BT = false, bool AT = false>
static int launch_one(cudaStream_t st, int sm_count, const CUtensorMap &tmA, const CUtensorMap &tmB, const StoreMaps &cm, GemmParams p)
{
    using Cfg = TileCfg<BN, DT, BT, AT>;
    p.tiles_m = (p.M + BM - 1) / BM;
    p.tiles_n = (p.N + BN - 1) / BN;
    p.num_kb = (p.K + Cfg::kBKE - 1) / Cfg::kBKE;
    if (p.group_m <= 0) p.group_m = 8;
    const long long total = (long long)p.batch * p.tiles_m * p.tiles_n;
    if (total <= 0) return BTM_OK;
    if (total > 0x3FFFFFFFLL) return set_error(BTM_ERR_UNSUPPORTED, "too many output tiles (%lld)", total);
    // Tail: r = total mod SMs tiles would leave most SMs idle for a whole tile time; when 2r <= SMs
    // they run as 2r half-width tiles instead (16-bit kernels with at least 128-column halves).
    int tail_big = 0;
    const int rem = (int)(total % sm_count);
    if (Cfg::kBMnMajor && BN >= 256 && rem > 0 && 2 * rem <= sm_count) tail_big = rem;
    p.tiles_full = (int)total - tail_big;
    p.tiles_tail = 2 * tail_big;
    const long long sched = (long long)p.tiles_full + p.tiles_tail;
    const int grid = (int)(sched < sm_count ? sched : sm_count);
    {
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3((unsigned)grid, 1, 1);
        cfg.blockDim = dim3(NUM_THREADS, 1, 1);
        cfg.dynamicSmemBytes = Cfg::kSmemBytes;
        cfg.stream = st;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr.val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        return check_cuda(cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, DT, BT, AT>, tmA, tmB, cm, p), "gemm_tc launch");
    }
}

template <int BN, int DT, bool BT = false, bool AT = false>
static cudaError_t raise_smem()
{
    return cudaFuncSetAttribute(gemm_tc_kernel<BN, DT, BT, AT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                TileCfg<BN, DT, BT, AT>::kSmemBytes);
}

int configure_gemm_tc_kernels()
{
    cudaError_t e = cudaSuccess;
    if (e == cudaSuccess) e = raise_smem<256, BTM_F16>();
    if (e == cudaSuccess) e = raise_smem<256, BTM_BF16>();
    if (e == cudaSuccess) e = raise_smem<128, BTM_F16>();
    if (e == cudaSuccess) e = raise_smem<128, BTM_BF16>();
    if (e == cudaSuccess) e = raise_smem<128, BTM_F32>();
    if (e == cudaSuccess) e = raise_smem<64, BTM_F32>();
    if (e == cudaSuccess) e = raise_smem<256, BTM_F16, true>();
    if (e == cudaSuccess) e = raise_smem<256, BTM_BF16, true>();
    if (e == cudaSuccess) e = raise_smem<128, BTM_F16, true>();
    if (e == cudaSuccess) e = raise_smem<128, BTM_BF16, true>();
    if (e == cudaSuccess) e = raise_smem<256, BTM_F16, false, true>();
    if (e == cudaSuccess) e = raise_smem<256, BTM_BF16, false, true>();
    if (e == cudaSuccess) e = raise_smem<128, BTM_F16, false, true>();
    if (e == cudaSuccess) e = raise_smem<128, BTM_BF16, false, true>();
    if (e == cudaSuccess) e = raise_smem<256, BTM_F16, true, true>();
    if (e == cudaSuccess) e = raise_smem<256, BTM_BF16, true, true>();
    if (e == cudaSuccess) e = raise_smem<128, BTM_F16, true, true>();
    if (e == cudaSuccess) e = raise_smem<128, BTM_BF16, true, true>();
    return check_cuda(e, "cudaFuncSetAttribute(gemm_tc)");
}

int launch_gemm_tc(int dtype, cudaStream_t st, int sm_count, const CUtensorMap &tmA, const CUtensorMap &tmB, const StoreMaps &cm,
                   const GemmParams &p, int force_bn)
{
    // Tile width: 256 columns unless the output is so small that narrower tiles are needed to
    // give every SM work.
    if (dtype == BTM_F32) {
        int bn = force_bn ? force_bn : 128;
        if (!force_bn) {
            const long long t128 = (long long)p.batch * ((p.M + BM - 1) / BM) * ((p.N + 127) / 128);
            if (t128 < sm_count) bn = 64;
        }
        if (bn == 64) return launch_one<64, BTM_F32>(st, sm_count, tmA, tmB, cm, p);
        return launch_one<128, BTM_F32>(st, sm_count, tmA, tmB, cm, p);
    }
    int bn = force_bn ? force_bn : 256;
    if (!force_bn) {
        const long long t256 = (long long)p.batch * ((p.M + BM - 1) / BM) * ((p.N + 255) / 256);
        if (t256 < sm_count) bn = 128;
    }
    if (dtype == BTM_F16) {
        if (bn == 128) return launch_one<128, BTM_F16>(st, sm_count, tmA, tmB, cm, p);
        return launch_one<256, BTM_F16>(st, sm_count, tmA, tmB, cm, p);
    }
    if (bn == 128) return launch_one<128, BTM_BF16>(st, sm_count, tmA, tmB, cm, p);
    return launch_one<256, BTM_BF16>(st, sm_count, tmA, tmB, cm, p);
}

// 16-bit product with operands in either storage order: a_t: A is stored [K,M] (tensor map dims (M, K), box 64 x 64);
// b_t: B is stored [N,K] (K-major; tensor map dims (K, N), box 64 x bn, so the caller fixes bn = 256 or 128).
int launch_gemm_tc_layout(int dtype, cudaStream_t st, int sm_count, const CUtensorMap &tmA, const CUtensorMap &tmB, const StoreMaps &cm,
                          const GemmParams &p, int bn, bool a_t, bool b_t)
{
#define BTM_LAYOUT_CASE(BTV, ATV)                                                                      \
    do {                                                                                               \
        if (dtype == BTM_F16) {                                                                        \
            if (bn == 128) return launch_one<128, BTM_F16, BTV, ATV>(st, sm_count, tmA, tmB, cm, p);   \
            return launch_one<256, BTM_F16, BTV, ATV>(st, sm_count, tmA, tmB, cm, p);                  \
        }                                                                                              \
        if (bn == 128) return launch_one<128, BTM_BF16, BTV, ATV>(st, sm_count, tmA, tmB, cm, p);      \
        return launch_one<256, BTM_BF16, BTV, ATV>(st, sm_count, tmA, tmB, cm, p);                     \
    } while (0)
    if (a_t && b_t) BTM_LAYOUT_CASE(true, true);
    if (a_t) BTM_LAYOUT_CASE(false, true);
    if (b_t) BTM_LAYOUT_CASE(true, false);
    BTM_LAYOUT_CASE(false, false);
#undef BTM_LAYOUT_CASE
}

// 16-bit product with B given transposed ([N,K] row-major, i.e. K-major): C = A . Bt^T. The B box of
// the tensor map is one whole tile (bn rows x 64 k), so the caller fixes bn (256 or 128).
int launch_gemm_tc_bt(int dtype, cudaStream_t st, int sm_count, const CUtensorMap &tmA, const CUtensorMap &tmB, const StoreMaps &cm,
                      const GemmParams &p, int bn)
{
    if (dtype == BTM_F16) {
        if (bn == 128) return launch_one<128, BTM_F16, true>(st, sm_count, tmA, tmB, cm, p);
        return launch_one<256, BTM_F16, true>(st, sm_count, tmA, tmB, cm, p);
    }
    if (bn == 128) return launch_one<128, BTM_BF16, true>(st, sm_count, tmA, tmB, cm, p);
    return launch_one<256, BTM_BF16, true>(st, sm_count, tmA, tmB, cm, p);
}

} // namespace btm
