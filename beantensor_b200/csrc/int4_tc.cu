// int4 weight-only matmul on the tensor cores for 8 < M <= 128 rows per pass:
//   out[m, n] = sum_k act[m, k] * dq[n, k],   dq[n, k] = f16_rne(float(W[n, k]) * float(S[n, k / group]))
// i.e. the weights are dequantised exactly as btm_int4_dequant defines them and the product runs as an
// fp16 tcgen05 matmul with fp32 accumulation in tensor memory.
//
// One CTA owns 64 weight rows (output columns) and all activation rows of the pass. Per 64-k block:
//   warp 0      TMA: the packed weights arrive as 256-k chunks (64 rows x 128 B, 128-byte swizzle) in
//               a small ring; the activation tile (BM rows x 64 k, K-major, 128-byte swizzle) goes
//               straight into the operand stage;
//   warps 2-5   dequantise: one 128-bit shared load (32 nibbles) per thread and block, unpack to exact
//               fp16 integers in natural k order, multiply by the group scale, and write the
//               64 x 64 fp16 tile in the K-major 128-byte-swizzled layout the tensor core reads;
//   warp 1      issues tcgen05.mma (M = 128, N = 64, both operands K-major) once both halves of the
//               stage are ready; tcgen05.commit frees the stage.
// After the last block warps 2-5 drain the accumulator with the shared TMA-store epilogue; rows past M
// are clipped by the store. The HBM traffic is the packed weights once (N*K/2 bytes) plus scales;
// activations are re-read per CTA from L2 (N/64 x M x K x 2 bytes).
//
// Measured (N=11008, K=4096, M=64): 43 us with HBM 6.5 % and the tensor pipe 12 % busy. The time follows
// the depth of the activation ring (3 stages 73 us, 4 stages 50 us, 8 stages 43 us) and not the number of
// proxy fences or hand-offs per chunk (one per 256-k chunk instead of four: no gain), the K order per CTA,
// or the dequantisation arithmetic (removed: 37 us): the 64-row x 128-byte activation tiles, which every
// CTA re-reads from L2, arrive with microseconds of latency, and with two CTAs per SM there is no shared
// memory left for a deeper ring. Fewer, wider CTAs (more weight rows per activation tile) are the way out.
#include <cuda_fp16.h>

#include "btm_internal.h"
#include "btm_ptx.cuh"
#include "gemm_epilogue.cuh"

namespace btm {

namespace i4tc {
constexpr int BN = 64;            // weight rows per CTA = UMMA N
constexpr int BKE = 64;           // k per operand stage
constexpr int CHUNK_K = 256;      // k per raw-weight chunk (128 bytes per row)
constexpr int RAW_BYTES = BN * 128;
constexpr int RAW_STAGES = 2;
constexpr int A_STAGES = 8; // activation tiles in flight (they come from L2 with about a microsecond of latency); the
                            // dequantised-weight ring is fed locally and stays short
constexpr int B_STAGES = 3;
constexpr int B_BYTES = BN * 128; // dequantised tile: 64 rows x 64 k fp16
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 64;
template <int BMR> // activation rows loaded per stage: 64 or 128
struct Cfg {
    static constexpr int A_BYTES = BMR * 128;
    // The tensor core always reads 128 rows of A. With BMR = 64 the upper half of that read falls on the
    // next activation tile (or, for the last one, on the B ring, which follows); it only feeds accumulator
    // rows 64..127, which are never stored.
    static constexpr int A_RING_BYTES = A_STAGES * A_BYTES;
    static constexpr int B_RING_BYTES = B_STAGES * B_BYTES;
    // The epilogue staging (16 KB) reuses the raw-weight ring, which is dead once the main loop is over.
    static_assert(RAW_STAGES * RAW_BYTES >= EPI_SMEM_BYTES / 2, "epilogue staging must fit in the raw ring");
    static constexpr int SMEM_BYTES = RAW_STAGES * RAW_BYTES + A_RING_BYTES + B_RING_BYTES + 1024; // + BN*G*2 bytes of scales at run time
};
} // namespace i4tc

__device__ __forceinline__ uint32_t i4_and_xor(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); // (a & b) ^ c
    return r;
}

// 8 two's-complement nibbles of a word -> 8 fp16 values v*s (one rounding each) in natural k order.
__device__ __forceinline__ uint4 dequant_word(uint32_t x, __half2 s2)
{
    const __half2 mul = __halves2half2(__ushort_as_half((unsigned short)0x3C00), __ushort_as_half((unsigned short)0x2C00)); // {1, 1/16}
    const __half2 add = __halves2half2(__ushort_as_half((unsigned short)0xE408), __ushort_as_half((unsigned short)0xD480)); // {-1032, -72}
    const uint32_t y = __byte_perm(x, x, 0x1010);
    const uint32_t z = __byte_perm(x, x, 0x3232);
    uint32_t p01 = i4_and_xor(y, 0x00F0000Fu, 0x64806408u);
    uint32_t p23 = i4_and_xor(y >> 8, 0x00F0000Fu, 0x64806408u);
    uint32_t p45 = i4_and_xor(z, 0x00F0000Fu, 0x64806408u);
    uint32_t p67 = i4_and_xor(z >> 8, 0x00F0000Fu, 0x64806408u);
    __half2 r0 = __hmul2(__hfma2(*reinterpret_cast<__half2 *>(&p01), mul, add), s2);
    __half2 r1 = __hmul2(__hfma2(*reinterpret_cast<__half2 *>(&p23), mul, add), s2);
    __half2 r2 = __hmul2(__hfma2(*reinterpret_cast<__half2 *>(&p45), mul, add), s2);
    __half2 r3 = __hmul2(__hfma2(*reinterpret_cast<__half2 *>(&p67), mul, add), s2);
    return make_uint4(*reinterpret_cast<uint32_t *>(&r0), *reinterpret_cast<uint32_t *>(&r1), *reinterpret_cast<uint32_t *>(&r2),
                      *reinterpret_cast<uint32_t *>(&r3));
}

template <int BMR>
__global__ void __launch_bounds__(i4tc::THREADS, 2)
int4_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmAct, const __grid_constant__ CUtensorMap tmW,
                    const __grid_constant__ StoreMaps cmaps, const GemmParams p, const __half *__restrict__ scales, int group,
                    int m_base)
{
    using namespace i4tc;
    using C = Cfg<BMR>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_raw_full[RAW_STAGES], bar_raw_empty[RAW_STAGES];
    __shared__ __align__(8) uint64_t bar_a_full[A_STAGES], bar_a_empty[A_STAGES], bar_b_full[B_STAGES], bar_b_empty[B_STAGES];
    __shared__ __align__(8) uint64_t bar_acc_full;
    __shared__ uint32_t tmem_base_holder;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t raw_base = smem_base;
    const uint32_t a_ring = smem_base + RAW_STAGES * RAW_BYTES;
    const uint32_t b_ring = a_ring + C::A_RING_BYTES;
    const uint32_t epi_base = raw_base; // reused after the main loop
    // scales of the CTA's 64 rows, [row][G] fp16, behind the epilogue staging area
    __half *sc_s = reinterpret_cast<__half *>(smem_raw + (b_ring + C::B_RING_BYTES - smem_u32(smem_raw)));
    const int n0 = blockIdx.x * BN;
    const int nkb = (p.K + BKE - 1) / BKE;
    const int nchunks = (p.K + CHUNK_K - 1) / CHUNK_K;
    // Every CTA walks K starting at a different chunk: all CTAs read the same activations, and in lock step
    // they would all ask the same L2 lines at the same moment (measured: 2 TB/s instead of the L2 rate).
    const int c_first = (int)(blockIdx.x % (unsigned)nchunks);

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < RAW_STAGES; ++i) {
            mbar_init(smem_u32(&bar_raw_full[i]), 1);
            mbar_init(smem_u32(&bar_raw_empty[i]), 4);
        }
        for (int i = 0; i < A_STAGES; ++i) {
            mbar_init(smem_u32(&bar_a_full[i]), 1);
            mbar_init(smem_u32(&bar_a_empty[i]), 1);
        }
        for (int i = 0; i < B_STAGES; ++i) {
            mbar_init(smem_u32(&bar_b_full[i]), 4);
            mbar_init(smem_u32(&bar_b_empty[i]), 1);
        }
        mbar_init(smem_u32(&bar_acc_full), 1);
        fence_mbar_init();
        prefetch_tmap(&tmAct);
        prefetch_tmap(&tmW);
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(&tmem_base_holder), TMEM_COLS);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_holder;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int rs = 0, os = 0;
            uint32_t rphase = 0, ophase = 0;
            bool ok = true;
            for (int ci = 0; ok && ci < nchunks; ++ci) {
                const int c = (c_first + ci) % nchunks;
                if (!mbar_wait(smem_u32(&bar_raw_empty[rs]), rphase ^ 1u, &abort_flag, p.status, WAIT_PRODUCER_EMPTY)) break;
                mbar_expect_tx(smem_u32(&bar_raw_full[rs]), RAW_BYTES);
                tma_load_3d(raw_base + rs * RAW_BYTES, &tmW, c * (CHUNK_K / 2), n0, 0, smem_u32(&bar_raw_full[rs]));
                if (++rs == RAW_STAGES) { rs = 0; rphase ^= 1u; }
                const int kb_end = min(nkb, (c + 1) * (CHUNK_K / BKE));
                for (int kb = c * (CHUNK_K / BKE); kb < kb_end; ++kb) {
                    if (!mbar_wait(smem_u32(&bar_a_empty[os]), ophase ^ 1u, &abort_flag, p.status, WAIT_PRODUCER_EMPTY)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(smem_u32(&bar_a_full[os]), C::A_BYTES);
                    tma_load_3d(a_ring + os * C::A_BYTES, &tmAct, kb * BKE, m_base, 0, smem_u32(&bar_a_full[os]));
                    if (++os == A_STAGES) { os = 0; ophase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(0u /*F16*/, false, false, 128, BN);
            int os = 0, bs = 0;
            uint32_t ophase = 0, bphase = 0;
            bool ok = true;
            bool first = true;
            for (int ci = 0; ok && ci < nchunks; ++ci) {
                const int c = (c_first + ci) % nchunks;
                const int kb_end = min(nkb, (c + 1) * (CHUNK_K / BKE));
                for (int kb = c * (CHUNK_K / BKE); kb < kb_end; ++kb) {
                    if (!mbar_wait_short(smem_u32(&bar_a_full[os]), ophase, &abort_flag, p.status, WAIT_MMA_FULL) ||
                        !mbar_wait_short(smem_u32(&bar_b_full[bs]), bphase, &abort_flag, p.status, WAIT_MMA_FULL)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a0 = a_ring + os * C::A_BYTES, b0 = b_ring + bs * B_BYTES;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t ad = make_smem_desc_sw128(a0 + ks * 32, 16, 1024);
                        const uint64_t bd = make_smem_desc_sw128(b0 + ks * 32, 16, 1024);
                        umma<1, false>(tmem_base, ad, bd, idesc, first ? 0u : 1u);
                        first = false;
                    }
                    umma_commit(smem_u32(&bar_a_empty[os])); // both tiles are free once these MMAs have read them
                    umma_commit(smem_u32(&bar_b_empty[bs]));
                    if (++os == A_STAGES) { os = 0; ophase ^= 1u; }
                    if (++bs == B_STAGES) { bs = 0; bphase ^= 1u; }
                }
            }
            if (ok) umma_commit(smem_u32(&bar_acc_full));
        }
    } else {
        // ------------------------------------------------------------ dequantise (warps 2..5), then epilogue
        const int dq = threadIdx.x - 64;     // 0..127
        const int row = dq >> 1, hsel = dq & 1; // weight row in the tile, which 32-k half of the block
        const int G = p.K / group;
        // The four dequantising warps fetch the tile's scales together, right away (a load issued once the
        // weight stream is queued would come back last), and meet on a named barrier of their own.
        for (int i = dq; i < BN * G; i += 128) sc_s[i] = __ldg(scales + min((size_t)n0 * G + i, (size_t)p.N * G - 1));
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const __half *srow = sc_s + row * G;
        const int gdiv = group / BKE; // k-blocks per scale group (group is a multiple of 64)
        const uint32_t swz = (uint32_t)(row & 7);
        int rs = 0, os = 0;
        uint32_t rphase = 0, ophase = 0;
        bool ok = true;
        for (int ci = 0; ok && ci < nchunks; ++ci) {
            const int c = (c_first + ci) % nchunks;
            ok = mbar_wait_short_warp(smem_u32(&bar_raw_full[rs]), rphase, &abort_flag, p.status, WAIT_EPI_STAGE);
            if (!ok) break;
            const uint32_t raw_row = raw_base + rs * RAW_BYTES + (uint32_t)row * 128u;
            const int kb_first = c * (CHUNK_K / BKE);
            const int nq = min(nkb, kb_first + CHUNK_K / BKE) - kb_first; // k-blocks in this chunk (1..4)
            // All packed words of the chunk are fetched and dequantised first (four independent instruction
            // streams for the scheduler to interleave); the stage hand-offs follow.
            uint4 d[CHUNK_K / BKE][4];
#pragma unroll
            for (int q = 0; q < CHUNK_K / BKE; ++q) {
                if (q < nq) {
                    uint4 pw; // packed 16 bytes = 32 nibbles: k = (kb_first + q)*64 + hsel*32 .. +32 of this row
                    const uint32_t src = raw_row + ((((uint32_t)(q * 2 + hsel)) ^ swz) << 4);
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(pw.x), "=r"(pw.y), "=r"(pw.z), "=r"(pw.w) : "r"(src));
                    const int kb = kb_first + q;
                    const __half2 s2 = __half2half2(srow[gdiv == 2 ? (kb >> 1) : (gdiv == 1 ? kb : kb / gdiv)]);
                    d[q][0] = dequant_word(pw.x, s2);
                    d[q][1] = dequant_word(pw.y, s2);
                    d[q][2] = dequant_word(pw.z, s2);
                    d[q][3] = dequant_word(pw.w, s2);
                }
            }
            // The raw chunk is in registers now: hand the buffer back before the (possibly waiting) stores.
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_raw_empty[rs]));
#pragma unroll
            for (int q = 0; q < CHUNK_K / BKE; ++q) {
                if (q < nq) {
                    ok = mbar_wait_short_warp(smem_u32(&bar_b_empty[os]), ophase ^ 1u, &abort_flag, p.status, WAIT_EPI_STAGE);
                    if (!ok) break;
                    const uint32_t brow = b_ring + os * B_BYTES + (uint32_t)row * 128u;
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        st_shared_v4(brow + ((((uint32_t)(hsel * 4 + j)) ^ swz) << 4), d[q][j].x, d[q][j].y, d[q][j].z, d[q][j].w);
                    fence_proxy_async_smem(); // generic-proxy writes -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar_b_full[os]));
                    if (++os == B_STAGES) { os = 0; ophase ^= 1u; }
                }
            }
            if (++rs == RAW_STAGES) { rs = 0; rphase ^= 1u; }
        }
        if (ok && mbar_wait_warp(smem_u32(&bar_acc_full), 0u, &abort_flag, p.status, WAIT_EPI_TMEM_FULL)) {
            tc_fence_after();
            const int quad = warp & 3;
            uint32_t epi_tiles = 0;
            // One staging tile per warp (64 output columns = one tile), carved from the epilogue area.
            epilogue_band<BTM_F16>(p, cmaps, tmem_base + ((uint32_t)(quad * 32) << 16), m_base + quad * 32, n0, BN, 0,
                                   epi_base + (uint32_t)quad * EPI_TILE_BYTES, epi_tiles, lane);
            epilogue_drain(lane);
        }
    }

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
    cudaError_t e = cudaFuncSetAttribute(int4_gemm_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, i4tc::Cfg<64>::SMEM_BYTES + 8192);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(int4_gemm_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, i4tc::Cfg<128>::SMEM_BYTES + 8192);
    return check_cuda(e, "cudaFuncSetAttribute(int4_gemm_tc)");
}

// Preconditions (checked by the caller): K % 128 == 0, group % 64 == 0, act / w / out 16-byte aligned,
// N % 8 == 0 (output pitch), M > 0.
int launch_int4_gemm_tc(cudaStream_t st, int M, int N, int K, int group, const void *act, const void *w, const void *scales, void *out,
                        int *status)
{
    using namespace i4tc;
    CUtensorMap tmAct, tmW;
    int rc = encode_tmap_3d(&tmW, BTM_U8, w, (uint64_t)K / 2, (uint64_t)N, 1, (uint64_t)K / 2, (uint64_t)K / 2, 128, BN);
    if (rc) return rc;
    for (int m_base = 0; m_base < M; m_base += 128) {
        const int rows = M - m_base < 128 ? M - m_base : 128;
        const int bmr = rows <= 64 ? 64 : 128;
        rc = encode_tmap_3d(&tmAct, BTM_F16, act, (uint64_t)K, (uint64_t)M, 1, (uint64_t)K * 2, (uint64_t)K * 2, 64, (uint32_t)bmr);
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
        p.c_vec_ok = 1;
        p.status = status;
        StoreMaps cm;
        rc = encode_store_maps(&cm, BTM_F16, p);
        if (rc) return rc;
        const unsigned grid = (unsigned)((N + BN - 1) / BN);
        const size_t sc_bytes = (size_t)BN * (K / group) * 2;
        if (bmr == 64)
            int4_gemm_tc_kernel<64><<<grid, THREADS, Cfg<64>::SMEM_BYTES + sc_bytes, st>>>(tmAct, tmW, cm, p, (const __half *)scales, group, m_base);
        else
            int4_gemm_tc_kernel<128><<<grid, THREADS, Cfg<128>::SMEM_BYTES + sc_bytes, st>>>(tmAct, tmW, cm, p, (const __half *)scales, group, m_base);
        rc = check_cuda(cudaGetLastError(), "int4 tensor-core matmul launch");
        if (rc) return rc;
    }
    return BTM_OK;
}

} // namespace btm
