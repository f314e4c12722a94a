// Epilogue of the tensor-core matmul kernels: accumulator (tensor memory) -> output type -> C.
//
// Fast path (C base, pitch and column offset 16-byte aligned): every epilogue warp owns a 32-row
// band of the tile. It reads 32 accumulator columns at a time with tcgen05.ld, rounds to the output
// type and writes them into a warp-private shared-memory tile of 32 rows x 128 bytes laid out with
// the 128-byte swizzle (conflict-free 16-byte stores); one lane then hands the tile to a TMA store
// (cp.async.bulk.tensor ... global.shared::cta). The TMA unit clips
// rows and columns beyond the matrix, so the band needs no predicates, and C is written in whole
// 128-byte lines. Two tiles per warp alternate so that a store drains while the next is filled. With
// several destination copies of C the peers are written by epilogue_band_multi (below).
// General path (unaligned C): per-thread row stores, as the kernels did originally.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "btm_internal.h"
#include "btm_ptx.cuh"

namespace btm {

constexpr int EPI_TILE_BYTES = 32 * 128;           // one staging tile: 32 rows x 128 B
constexpr int EPI_WARP_BYTES = 2 * EPI_TILE_BYTES; // two tiles per epilogue warp
constexpr int EPI_SMEM_BYTES = 4 * EPI_WARP_BYTES; // four epilogue warps

__device__ __forceinline__ void tma_store_3d(const CUtensorMap *m, uint32_t src_smem, int x, int y, int z)
{
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(m), "r"(src_smem), "r"(x),
                 "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's bulk groups still have to READ their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// 16 bytes to a multicast address: the switch writes them at the same offset of every memory bound to the object.
__device__ __forceinline__ void multimem_st_v4(void *mc_addr, const uint4 &v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}

template <int DT>
__device__ __forceinline__ void pack16(const uint32_t (&acc)[32], uint32_t (&packed)[16])
{
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const float lo = __uint_as_float(acc[2 * j]), hi = __uint_as_float(acc[2 * j + 1]);
        if constexpr (DT == BTM_F16) {
            __half2 h = __floats2half2_rn(lo, hi);
            packed[j] = *reinterpret_cast<uint32_t *>(&h);
        } else {
            __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
            packed[j] = *reinterpret_cast<uint32_t *>(&h);
        }
    }
}

// Fused bias and activation on 32 accumulator columns (col .. col + 31) of this lane's row: lane j fetches
// bias[col + j] once and the values go round the warp by shuffle. Nothing is done (one uniform branch) when
// the launch has neither.
template <int DT>
__device__ __forceinline__ void bias_act(const GemmParams &p, uint32_t (&v)[32], int col, int lane)
{
    if (p.bias == nullptr && p.act == 0) return;
    float b = 0.0f;
    if (p.bias != nullptr && col + lane < p.N) {
        if constexpr (DT == BTM_F32) b = __ldg(reinterpret_cast<const float *>(p.bias) + col + lane);
        else if constexpr (DT == BTM_F16) b = __half2float(__ldg(reinterpret_cast<const __half *>(p.bias) + col + lane));
        else b = __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16 *>(p.bias) + col + lane));
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        float x = __uint_as_float(v[j]) + __shfl_sync(0xffffffffu, b, j);
        if (p.act == 1) x = fmaxf(x, 0.0f);
        v[j] = __float_as_uint(x);
    }
}

// Debug bounds check of a hand-computed store: elements [off, off + n) from a C base. False (and the code in the status
// word) when the launch was started with bounds checks on and the range leaves the output; the caller skips the store.
__device__ __forceinline__ bool store_in_bounds(const GemmParams &p, long long off, int n)
{
    if (!p.debug_bounds) return true;
    if (off >= 0 && off + n <= p.c_extent) return true;
    atomicCAS(p.status, 0, (int)BOUNDS_STORE);
    return false;
}

// Per-thread stores of 32 consecutive columns of one output row (general path).
template <int DT>
__device__ __forceinline__ void store_row_direct(const GemmParams &p, const uint32_t (&acc)[32], long long elem_off, int ncols_valid)
{
    if (!store_in_bounds(p, elem_off, ncols_valid)) return;
    if constexpr (DT == BTM_F32) {
        for (int d = 0; d < p.ndst; ++d) {
            float *dst = reinterpret_cast<float *>(p.C[d]) + elem_off;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols_valid) dst[j] = __uint_as_float(acc[j]);
        }
    } else {
        uint32_t packed[16];
        pack16<DT>(acc, packed);
        for (int d = 0; d < p.ndst; ++d) {
            uint16_t *dst = reinterpret_cast<uint16_t *>(p.C[d]) + elem_off;
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j < ncols_valid) dst[j] = (uint16_t)((j & 1) ? (packed[j >> 1] >> 16) : (packed[j >> 1] & 0xFFFFu));
        }
    }
}

// Band drain when C has several destination copies (the fused all-gather of the N-sharded product).
// 128 output columns at a time: both staging tiles are filled, the local copy goes out as two TMA
// stores, and the peers are written with plain 16-byte stores from registers, laid out so that one
// warp instruction covers two rows x 256 contiguous bytes. Peer traffic crosses NVLink, where 256-byte
// contiguous writes pack better than the 128-byte rows of a staging tile, and stores from registers
// are posted: the warp never waits for a peer before it frees the accumulator.
template <int DT>
__device__ __forceinline__ void epilogue_band_multi(const GemmParams &p, const StoreMaps &cmaps, uint32_t tmem_band, int row0,
                                                    int col_first, int bn, int batch, uint32_t epi_smem, uint32_t &tile_count, int lane)
{
    const uint32_t swz = (uint32_t)(lane & 7);
    // Pacing: the peer stores of this tile are issued in (bn / 128) x (ndst - 1) batches, batch j not
    // before t0 + j x step, so that they leave the SM spread over the time the next tile's main loop
    // takes instead of as one burst.
    const long long t0 = clock64();
    const long long step = p.pace_cycles > 0 ? (long long)p.pace_cycles / ((bn / 128) * (p.ndst - 1)) : 0;
    int batch_no = 0;
#pragma unroll 1
    for (int c = 0; c < bn / 128; ++c) {
        tile_count += 2;
        // Both staging tiles are about to be rewritten: the local stores of the previous pair must have read them.
        if (lane == 0) bulk_wait_read<0>();
        __syncwarp();
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const uint32_t row_addr = epi_smem + (uint32_t)t * EPI_TILE_BYTES + (uint32_t)lane * 128u;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t v[32], q[16];
                tmem_ld_32x32(tmem_band + (uint32_t)(c * 128 + t * 64 + h * 32), v);
                tmem_ld_wait();
                bias_act<DT>(p, v, col_first + c * 128 + t * 64 + h * 32, lane);
                pack16<DT>(v, q);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    st_shared_v4(row_addr + (((uint32_t)(h * 4 + j) ^ swz) << 4), q[4 * j], q[4 * j + 1], q[4 * j + 2], q[4 * j + 3]);
            }
        }
        fence_proxy_async_smem();
        __syncwarp();
        const int col = col_first + c * 128;
        // With a multicast mapping the local copy is written by the same multimem stores as the peers' (this device
        // is a member of the object), so the staging tiles only serve the transposition below.
        if (lane == 0 && p.mc == nullptr) {
            if (row0 < p.M && col < p.N) tma_store_3d(&cmaps.m[0], epi_smem, (int)p.col0 + col, row0, batch);
            if (row0 < p.M && col + 64 < p.N) tma_store_3d(&cmaps.m[0], epi_smem + EPI_TILE_BYTES, (int)p.col0 + col + 64, row0, batch);
            bulk_commit();
        }
        // Peers: lane l owns the 16-byte chunk (l & 15) of the 256-byte row pieces of rows 2 i + (l >> 4).
        const int chunk = lane & 15, tsel = chunk >> 3, cj = chunk & 7;
        uint4 regs[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int r = 2 * i + (lane >> 4);
            const uint32_t a = epi_smem + (uint32_t)tsel * EPI_TILE_BYTES + (uint32_t)r * 128u + ((((uint32_t)cj) ^ (uint32_t)(r & 7)) << 4);
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(regs[i].x), "=r"(regs[i].y), "=r"(regs[i].z), "=r"(regs[i].w) : "r"(a));
        }
        const int ccol = col + chunk * 8; // first of this lane's 8 columns
        const long long base = (long long)batch * p.strideC + p.col0 + ccol;
        if (p.mc != nullptr) {
            // One outbound copy: 16-byte multimem stores, two rows x 256 contiguous bytes per warp instruction. The
            // launcher guarantees that N is a multiple of 8 here, so a lane's 8 columns are all inside or all outside.
            uint16_t *dst = reinterpret_cast<uint16_t *>(p.mc);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int row = row0 + 2 * i + (lane >> 4);
                if (row < p.M && ccol + 8 <= p.N && store_in_bounds(p, base + (long long)row * p.ldc, 8))
                    multimem_st_v4(dst + base + (long long)row * p.ldc, regs[i]);
            }
            continue;
        }
        for (int d = 1; d < p.ndst; ++d, ++batch_no) {
            uint16_t *dst = reinterpret_cast<uint16_t *>(p.C[d]);
            if (step > 0) {
                const long long due = t0 + step * batch_no;
                while (clock64() < due) __nanosleep(256); // bounded: `due` is at most pace_cycles away
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int row = row0 + 2 * i + (lane >> 4);
                if (row < p.M && ccol < p.N && store_in_bounds(p, base + (long long)row * p.ldc, min(8, p.N - ccol))) {
                    uint16_t *q = dst + base + (long long)row * p.ldc;
                    if (ccol + 8 <= p.N) {
                        *reinterpret_cast<uint4 *>(q) = regs[i];
                    } else {
                        const uint32_t w[4] = {regs[i].x, regs[i].y, regs[i].z, regs[i].w};
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (ccol + e < p.N) q[e] = (uint16_t)((e & 1) ? (w[e >> 1] >> 16) : (w[e >> 1] & 0xFFFFu));
                    }
                }
            }
        }
    }
}

// Drains one 32-row band (this warp's tensor-memory quadrant) of a finished tile.
//   tmem_band   tensor-memory address of the band's first accumulator column (lane bits included)
//   row0        first output row of the band; col_first first output column of the tile; bn its width
//   epi_smem    this warp's two staging tiles (shared-memory address, 1024-byte aligned)
//   tile_count  running count of staging tiles this warp has used (selects the buffer)
template <int DT>
__device__ __forceinline__ void epilogue_band(const GemmParams &p, const StoreMaps &cmaps, uint32_t tmem_band, int row0, int col_first,
                                              int bn, int batch, uint32_t epi_smem, uint32_t &tile_count, int lane)
{
    constexpr int kColsPerTile = (DT == BTM_F32) ? 32 : 64; // 128 bytes of output per row
    if (!p.c_vec_ok) {
        const int row = row0 + lane;
        const long long row_off = (long long)batch * p.strideC + (long long)row * p.ldc + p.col0;
#pragma unroll 1
        for (int c = 0; c < bn / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_band + (uint32_t)(c * 32), v);
            tmem_ld_wait();
            const int col = col_first + c * 32;
            bias_act<DT>(p, v, col, lane);
            const int valid = min(32, p.N - col);
            if (row < p.M && valid > 0) store_row_direct<DT>(p, v, row_off + col, valid);
        }
        return;
    }
    const uint32_t swz = (uint32_t)(lane & 7);
    if constexpr (DT != BTM_F32) {
        if ((p.ndst > 1 || p.mc != nullptr) && (bn & 127) == 0) {
            epilogue_band_multi<DT>(p, cmaps, tmem_band, row0, col_first, bn, batch, epi_smem, tile_count, lane);
            return;
        }
    }
#pragma unroll 1
    for (int c = 0; c < bn / kColsPerTile; ++c) {
        const uint32_t buf = epi_smem + (tile_count & 1u) * EPI_TILE_BYTES;
        ++tile_count;
        // The store issued two tiles ago used this buffer: it must have finished reading it.
        if (lane == 0) bulk_wait_read<1>();
        __syncwarp();
        const uint32_t row_addr = buf + (uint32_t)lane * 128u;
        if constexpr (DT == BTM_F32) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_band + (uint32_t)(c * 32), v);
            tmem_ld_wait();
            bias_act<DT>(p, v, col_first + c * 32, lane);
#pragma unroll
            for (int j = 0; j < 8; ++j) st_shared_v4(row_addr + (((uint32_t)j ^ swz) << 4), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t v[32], q[16];
                tmem_ld_32x32(tmem_band + (uint32_t)(c * 64 + h * 32), v);
                tmem_ld_wait();
                bias_act<DT>(p, v, col_first + c * 64 + h * 32, lane);
                pack16<DT>(v, q);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    st_shared_v4(row_addr + (((uint32_t)(h * 4 + j) ^ swz) << 4), q[4 * j], q[4 * j + 1], q[4 * j + 2], q[4 * j + 3]);
            }
        }
        fence_proxy_async_smem(); // generic-proxy writes above -> visible to the TMA unit
        __syncwarp();
        const int col = col_first + c * kColsPerTile;
        if (lane == 0) {
            if (row0 < p.M && col < p.N) tma_store_3d(&cmaps.m[0], buf, (int)p.col0 + col, row0, batch);
            bulk_commit(); // an empty group when nothing was stored keeps the buffer accounting uniform
        }
    }
}

// Before the warp leaves the kernel: every store it issued has completed.
__device__ __forceinline__ void epilogue_drain(int lane)
{
    if (lane == 0) bulk_wait_all<0>();
    __syncwarp();
}

} // namespace btm
