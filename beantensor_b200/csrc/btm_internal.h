// Internal declarations shared by the translation units of libbtm.so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/btm.h"

namespace btm {

constexpr int kMaxDst = 8; // destinations of one epilogue store (ranks of a single NVSwitch box)

// Per-call description of a (batched) matmul for the tensor-core kernels.
struct GemmParams {
    int M, N, K;         // one product
    int batch;           // independent products (1 for plain matmul)
    int tiles_m, tiles_n; // tiles per product
    int num_kb;          // k-blocks per tile
    int tiles_full;      // two-SM kernel: tiles of full width in the list ...
    int tiles_tail;      // ... followed by this many half-width tiles
    int group_m;         // tile raster: m-tiles per L2 group
    void *C[kMaxDst];    // output bases; [0] is local, others are peer-mapped copies of C
    int ndst;
    long long ldc;     // elements
    long long strideC; // elements between products
    long long col0;    // first output column of this launch inside C
    void *mc;          // multicast mapping of C (one multimem store reaches every rank's copy), or NULL
    int pace_cycles;   // >0: peer stores of one tile are spread over this many SM cycles (several destinations only)
    const void *bias;  // optional: one value per output column (same dtype as C), added to the fp32 accumulator before rounding
    int act;           // 0 none, 1 ReLU (after the bias)
    int c_vec_ok;      // 16-byte vector stores into C are legal
    int *status;       // device status word (bounded waits report here)
    long long wait_limit; // SM cycles after which a wait inside the kernel gives up (set by fill_wait_params)
    int debug_skip_loads; // test hook: the producer warps issue no loads, so the consumers' waits run out
    // Debug bounds checks (BTM_DEBUG_BOUNDS=1 or btm_debug_set("bounds", 1)): every address that an epilogue computes by
    // hand from tile coordinates (the per-thread row stores, the peer stores and the multimem stores; TMA stores are
    // clipped by the hardware) is compared with the extent of C before it is used. A store that would fall outside is
    // skipped and code BOUNDS_STORE goes to the status word: the stand-in for a memory checker on this path.
    int debug_bounds;
    long long c_extent; // elements from a C base that this launch may touch: [0, c_extent)
};

// Output tensor maps of the epilogue's TMA stores, one per destination copy of C (local first, then peers).
struct StoreMaps {
    CUtensorMap m[kMaxDst];
};

// Per-device state, created once by btm_init.
struct DeviceState {
    std::atomic<bool> ready;
    int sm_count;
    int *status;        // device memory, one int
    cudaMemPool_t pool; // scratch of the fp32 split: allocated and freed in stream order, one block per call
};

int set_error(int code, const char *fmt, ...);
// Sets p->wait_limit (the default of about one second, or what btm_debug_set installed), the test hooks and, from
// the fields already set (M, N, batch, ldc, strideC, col0), the extent used by the debug bounds checks.
void fill_wait_params(GemmParams *p);
int check_cuda(cudaError_t e, const char *what);
DeviceState *device_state(int device); // NULL + error set on failure

// Encodes a rank-3 tiled tensor map (dims innermost first). swizzle: 0 none, 1 128-byte, 2 64-byte.
int encode_tmap_3d(CUtensorMap *out, int dtype, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                   uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, int swizzle = 1);

// Launchers (defined next to their kernels). All return a btm_status.
int launch_gemm_tc(int dtype, cudaStream_t st, int sm_count, const CUtensorMap &tmA, const CUtensorMap &tmB, const StoreMaps &cm,
                   const GemmParams &p, int force_bn);
int launch_gemm_tc_bt(int dtype, cudaStream_t st, int sm_count, const CUtensorMap &tmA, const CUtensorMap &tmB, const StoreMaps &cm,
                      const GemmParams &p, int bn);
int launch_gemm_tc_layout(int dtype, cudaStream_t st, int sm_count, const CUtensorMap &tmA, const CUtensorMap &tmB, const StoreMaps &cm,
                          const GemmParams &p, int bn, bool a_t, bool b_t);
// bias / act: see GemmParams. a_cs / b_cs: element stride between consecutive columns of A / B (1 = row-major).
int launch_gemm_simt(int dtype, cudaStream_t st, int batch, int M, int N, int K, const void *A, long long lda,
                     long long strideA, const void *B, long long ldb, long long strideB, void *C, long long ldc,
                     long long strideC, const void *bias = nullptr, int act = 0, long long a_cs = 1, long long b_cs = 1);
int launch_split_tf32(cudaStream_t st, const float *src, long long ld, int rows, int cols, float *dst_hi,
                      float *dst_lo, long long ld_dst);
int launch_split_tf32_pair(cudaStream_t st, const float *A, long long lda, int M, int K, float *a_hi, float *a_lo, const float *B,
                           long long ldb, int N, float *b_hi, float *b_lo, long long Kp);
int launch_split_tf32_transpose(cudaStream_t st, const float *src, long long ld, int rows, int cols, float *dst_hi,
                                float *dst_lo, long long ld_dst);
int launch_int4_gemv(cudaStream_t st, int sm_count, int M, int N, int K, int group, const void *act,
                     const void *w, const void *scales, void *out, int *status);
int launch_int4_dequant(cudaStream_t st, int N, int K, int group, const void *w, const void *scales, void *out);
int launch_int4_unpack(cudaStream_t st, int N, int K, const void *w, void *out);
int launch_convert(cudaStream_t st, int src_dtype, int dst_dtype, long long n, const void *src, void *dst);
int launch_int4_quantize(cudaStream_t st, int N, int K, int group, const void *w, void *packed, void *scales);
int configure_gemm_tc_kernels(); // raises dynamic shared-memory limits; once per device
int configure_gemm_tc2_kernels();
int configure_int4_tc_kernels();
int configure_int4_gemv_kernels();
int configure_int4_gemv_regs_kernels();
// Register-resident GEMV. Returns a btm_status, or -1 when the shape is outside what it takes (nothing launched).
int launch_int4_gemv_regs(cudaStream_t st, int sm_count, int M, int N, int K, int group, const void *act, const void *w,
                          const void *scales, void *out);
int launch_int4_gemm_tc(cudaStream_t st, int M, int N, int K, int group, const void *act, const void *w, const void *scales, void *out,
                        int *status, int sm_count);
int launch_gemm_tc2(int dtype, cudaStream_t st, int sm_count, const CUtensorMap &tmA, const CUtensorMap &tmB, const StoreMaps &cm,
                    const GemmParams &p);
// Fills `cm` for the destinations in `p` (no-op when p.c_vec_ok == 0: the general store path needs no maps).
int encode_store_maps(StoreMaps *cm, int dtype, const GemmParams &p);

} // namespace btm
