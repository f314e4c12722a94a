// C ABI of libbtm.so: argument checks, per-device state, tensor-map encoding and dispatch to the
// kernels. Nothing here computes on the CPU; every path ends in a CUDA launch or an error.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <atomic>
#include <mutex>

#include "btm_internal.h"

namespace btm {

static thread_local char g_err[512] = "";
static thread_local int g_code = BTM_OK;
static int last_code() { return g_code != BTM_OK ? g_code : BTM_ERR_CUDA; }

int set_error(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    g_code = code;
    return code;
}

int check_cuda(cudaError_t e, const char *what)
{
    if (e == cudaSuccess) return BTM_OK;
    // Same split as the reference's CUDA_CHECK_ERROR (Errors/Logic.h:50-59): allocation
    // failures are reported apart from every other runtime error.
    if (e == cudaErrorMemoryAllocation) return set_error(BTM_ERR_OOM, "CUDA Error: %s (%s)", cudaGetErrorString(e), what);
    return set_error(BTM_ERR_CUDA, "CUDA Error: %s (%s)", cudaGetErrorString(e), what);
}

// Test hooks (btm_debug_set): process-wide, read at every launch.
static std::atomic<long long> g_dbg_wait_limit{0};
static std::atomic<int> g_dbg_skip_loads{0};
static std::atomic<int> g_dbg_bounds{-1};            // -1: not decided yet (BTM_DEBUG_BOUNDS is read once)
static std::atomic<long long> g_dbg_bounds_shrink{0}; // test hook: pretend C is this many elements shorter

void fill_wait_params(GemmParams *p)
{
    const long long lim = g_dbg_wait_limit.load(std::memory_order_relaxed);
    p->wait_limit = lim > 0 ? lim : 2000000000LL; // about one second of SM clocks; the longest kernel here runs milliseconds
    p->debug_skip_loads = g_dbg_skip_loads.load(std::memory_order_relaxed);
    int b = g_dbg_bounds.load(std::memory_order_relaxed);
    if (b < 0) {
        const char *e = getenv("BTM_DEBUG_BOUNDS");
        b = (e && *e && strcmp(e, "0")) ? 1 : 0;
        g_dbg_bounds.store(b);
    }
    p->debug_bounds = b;
    const long long batches = p->batch > 1 ? p->batch : 1;
    p->c_extent = (batches - 1) * p->strideC + (long long)(p->M > 0 ? p->M - 1 : 0) * p->ldc + p->col0 + p->N -
                  g_dbg_bounds_shrink.load(std::memory_order_relaxed);
}

constexpr int kMaxDevices = 64;
static DeviceState g_dev[kMaxDevices];
static std::mutex g_dev_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static std::atomic<EncodeTiledFn> g_encode{nullptr};

// Looks the driver's tensor-map encoder up once per process. Allocates nothing.
static int ensure_encode()
{
    if (g_encode.load(std::memory_order_acquire)) return BTM_OK;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    int rc = check_cuda(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres), "cudaGetDriverEntryPoint");
    if (rc) return rc;
    if (qres != cudaDriverEntryPointSuccess || !fn) return set_error(BTM_ERR_CUDA, "CUDA Error: driver does not export cuTensorMapEncodeTiled");
    g_encode.store((EncodeTiledFn)fn, std::memory_order_release);
    return BTM_OK;
}

DeviceState *device_state(int device)
{
    if (device < 0 || device >= kMaxDevices) {
        set_error(BTM_ERR_INVALID, "Invalid GPU ID %d", device);
        return nullptr;
    }
    DeviceState *ds = &g_dev[device];
    // Ready path: no lock and no device query, only the switch of the calling thread's current device (the
    // reference's pool threads arrive with whatever device they used last).
    if (ds->ready.load(std::memory_order_acquire)) {
        if (check_cuda(cudaSetDevice(device), "cudaSetDevice")) return nullptr;
        return ds;
    }
    int count = 0;
    if (check_cuda(cudaGetDeviceCount(&count), "cudaGetDeviceCount")) return nullptr;
    if (device >= count) {
        set_error(BTM_ERR_INVALID, "Invalid GPU ID %d (device count %d)", device, count);
        return nullptr;
    }
    if (check_cuda(cudaSetDevice(device), "cudaSetDevice")) return nullptr;
    std::lock_guard<std::mutex> lock(g_dev_mu);
    if (ds->ready.load(std::memory_order_acquire)) return ds;
    cudaDeviceProp prop;
    if (check_cuda(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties")) return nullptr;
    if (prop.major != 10) {
        set_error(BTM_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major,
                  prop.minor);
        return nullptr;
    }
    if (ensure_encode()) return nullptr;
    if (check_cuda(cudaMalloc(&ds->status, sizeof(int)), "cudaMalloc(status)")) return nullptr;
    if (check_cuda(cudaMemset(ds->status, 0, sizeof(int)), "cudaMemset(status)")) return nullptr;
    // Scratch of the fp32 product comes from a pool of this library's own, in stream order. The release
    // threshold keeps freed blocks in the pool, so that after the first call of a shape an allocation is a
    // bookkeeping step on the host and not a trip to the driver.
    cudaMemPoolProps props;
    memset(&props, 0, sizeof(props));
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = device;
    if (check_cuda(cudaMemPoolCreate(&ds->pool, &props), "cudaMemPoolCreate")) return nullptr;
    unsigned long long keep = ~0ull;
    if (check_cuda(cudaMemPoolSetAttribute(ds->pool, cudaMemPoolAttrReleaseThreshold, &keep), "cudaMemPoolSetAttribute")) return nullptr;
    if (configure_gemm_tc_kernels()) return nullptr;
    if (configure_gemm_tc2_kernels()) return nullptr;
    if (configure_int4_tc_kernels()) return nullptr;
    if (configure_int4_gemv_kernels()) return nullptr;
    ds->sm_count = prop.multiProcessorCount;
    ds->ready.store(true, std::memory_order_release);
    return ds;
}

int encode_tmap_3d(CUtensorMap *out, int dtype, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                   uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0, uint32_t box1, int swizzle)
{
    CUtensorMapDataType dt = dtype == BTM_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                             : dtype == BTM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                             : dtype == BTM_U8   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                                 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    cuuint32_t box[3] = {box0, box1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (int rc = ensure_encode()) return rc;
    CUresult r = g_encode.load(std::memory_order_acquire)(out, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return set_error(BTM_ERR_CUDA, "CUDA Error: cuTensorMapEncodeTiled failed with code %d (dims %llu x %llu x %llu)", (int)r,
                         (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2);
    return BTM_OK;
}

int encode_store_maps(StoreMaps *cm, int dtype, const GemmParams &p)
{
    memset(cm, 0, sizeof(*cm));
    if (!p.c_vec_ok) return BTM_OK;
    const uint64_t es = dtype == BTM_F32 ? 4 : 2;
    const uint32_t box_cols = dtype == BTM_F32 ? 32 : 64; // 128 bytes per staged row
    const uint64_t width = (uint64_t)p.col0 + (uint64_t)p.N; // stores are clipped at the last column this launch owns
    const uint64_t s1 = (uint64_t)p.ldc * es;
    const uint64_t s2 = p.batch > 1 ? (uint64_t)p.strideC * es : s1;
    for (int d = 0; d < p.ndst; ++d) {
        int rc = encode_tmap_3d(&cm->m[d], dtype, p.C[d], width, (uint64_t)p.M, (uint64_t)p.batch, s1, s2, box_cols, 32);
        if (rc) return rc;
    }
    return BTM_OK;
}

static size_t es_of(int dtype) { return dtype == BTM_F32 ? 4 : 2; }
static bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

// Can TMA address this operand? Base and every pitch must be multiples of 16 bytes.
static bool tma_ok(const void *p, long long ld, long long stride, int batch, size_t es)
{
    if (!aligned16(p)) return false;
    if ((ld * (long long)es) % 16) return false;
    if (batch > 1 && (stride * (long long)es) % 16) return false;
    return true;
}

struct GemmCall {
    int dtype, batch, M, N, K;
    const void *A, *B;
    long long lda, ldb, strideA, strideB;
    void *C[kMaxDst];
    int ndst;
    void *mc; // multicast mapping of C, or NULL
    long long ldc, strideC, col0;
    const void *bias; // optional, one value per column of this launch's N
    int act;          // 0 none, 1 ReLU
};

static int run_16bit(DeviceState *ds, cudaStream_t st, const GemmCall &c)
{
    const size_t es = 2;
    const bool tc = c.K > 0 && tma_ok(c.A, c.lda, c.strideA, c.batch, es) && tma_ok(c.B, c.ldb, c.strideB, c.batch, es);
    if (!tc) {
        for (int d = 0; d < c.ndst; ++d) {
            int rc = launch_gemm_simt(c.dtype, st, c.batch, c.M, c.N, c.K, c.A, c.lda, c.strideA, c.B, c.ldb, c.strideB,
                                      (char *)c.C[d] + c.col0 * (long long)es, c.ldc, c.strideC, c.bias, c.act);
            if (rc) return rc;
        }
        return BTM_OK;
    }
    CUtensorMap tmA, tmB;
    const uint64_t sA = c.batch > 1 ? (uint64_t)c.strideA * es : (uint64_t)c.lda * es;
    const uint64_t sB = c.batch > 1 ? (uint64_t)c.strideB * es : (uint64_t)c.ldb * es;
    int rc = encode_tmap_3d(&tmA, c.dtype, c.A, (uint64_t)c.K, (uint64_t)c.M, (uint64_t)c.batch, (uint64_t)c.lda * es, sA, 64, 128);
    if (rc) return rc;
    rc = encode_tmap_3d(&tmB, c.dtype, c.B, (uint64_t)c.N, (uint64_t)c.K, (uint64_t)c.batch, (uint64_t)c.ldb * es, sB, 64, 64);
    if (rc) return rc;
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.M = c.M;
    p.N = c.N;
    p.K = c.K;
    p.batch = c.batch;
    p.group_m = 8;
    if (const char *gm = getenv("BTM_GROUP_M")) p.group_m = std::max(1, atoi(gm)); // tile raster: m-tiles per L2 group (tuning aid)
    p.ndst = c.ndst;
    bool vec = (c.ldc * (long long)es) % 16 == 0 && (c.col0 * (long long)es) % 16 == 0 &&
               (c.batch == 1 || (c.strideC * (long long)es) % 16 == 0);
    for (int d = 0; d < c.ndst; ++d) {
        p.C[d] = c.C[d];
        vec = vec && aligned16(c.C[d]);
    }
    p.ldc = c.ldc;
    p.strideC = c.strideC;
    p.col0 = c.col0;
    p.c_vec_ok = vec ? 1 : 0;
    p.status = ds->status;
    fill_wait_params(&p);
    p.bias = c.bias;
    p.act = c.act;
    p.mc = c.mc;
    if (c.ndst > 1) {
        // Peer stores of a tile are spread over part of the next tile's main loop instead of leaving the
        // SM as one burst. Unit: SM cycles per 64-deep k-block (a k-block of a 256 x 256 pair tile takes
        // 650-750). Measured on 16384^3 bf16: at 8 ranks 500 gives 1.05 ms against 1.12-1.22 ms unpaced
        // and 100-400 are no better than unpaced; at 4 ranks pacing does not help, so it is off below 8.
        // BTM_NSHARD_PACE overrides (0 = off).
        const char *pace = getenv("BTM_NSHARD_PACE");
        const long long per_kb = pace ? atoll(pace) : (c.ndst >= 8 ? 500 : 0);
        p.pace_cycles = (int)std::min<long long>(per_kb * ((c.K + 63) / 64), 1LL << 30);
    }
    // CTA pairs (256 x 256 tiles, B shared between two SMs) once there is enough work to fill a good
    // part of the machine; single CTAs (128 x 256 or 128 x 128) for small outputs.
    // BTM_FORCE_KERNEL=1cta|2cta overrides the choice (used by the tests to cover both on every shape).
    const long long pair_tiles = (long long)c.batch * ((c.M + 255) / 256) * ((c.N + 255) / 256);
    // Short products (K < 512, e.g. the batched 512x512x128 workload) stay on single CTAs: with two k-blocks
    // per tile the pair handshake costs more than the halved B traffic saves (12.1 vs 15.7 us measured).
    bool pair = c.M > 128 && pair_tiles >= ds->sm_count / 4 && c.K >= 512;
    if (const char *force = getenv("BTM_FORCE_KERNEL")) {
        if (!strcmp(force, "1cta")) pair = false;
        else if (!strcmp(force, "2cta")) pair = true;
    }
    StoreMaps cm;
    rc = encode_store_maps(&cm, c.dtype, p);
    if (rc) return rc;
    if (pair) return launch_gemm_tc2(c.dtype, st, ds->sm_count, tmA, tmB, cm, p);
    return launch_gemm_tc(c.dtype, st, ds->sm_count, tmA, tmB, cm, p, 0);
}

static int run_f32_planes(DeviceState *ds, cudaStream_t st, const GemmCall &c, float *a_hi, float *b_hi, long long Kp);

static int run_f32(DeviceState *ds, cudaStream_t st, const GemmCall &c, void *ws, size_t ws_bytes)
{
    // Operand planes in scratch: A_hi, A_lo [M, Kp] then B^T_hi, B^T_lo [N, Kp], pitch padded to 4 floats.
    const long long Kp = (c.K + 3) & ~3LL;
    const size_t a_plane = (size_t)c.M * Kp, b_plane = (size_t)c.N * Kp;
    const size_t need = (2 * a_plane + 2 * b_plane) * sizeof(float);
    if (c.K == 0 || c.M == 0 || c.N == 0)
        return launch_gemm_simt(BTM_F32, st, 1, c.M, c.N, c.K, c.A, c.lda, 0, c.B, c.ldb, 0, c.C[0], c.ldc, 0, c.bias, c.act);
    if (ws_bytes < need) return set_error(BTM_ERR_INVALID, "fp32 matmul: workspace of %zu bytes is smaller than the %zu needed", ws_bytes, need);
    float *a_hi = (float *)ws, *a_lo = a_hi + a_plane, *b_hi = a_lo + a_plane, *b_lo = b_hi + b_plane;
    int rc = launch_split_tf32_pair(st, (const float *)c.A, c.lda, c.M, c.K, a_hi, a_lo, (const float *)c.B, c.ldb, c.N, b_hi, b_lo, Kp);
    if (rc) return rc;
    return run_f32_planes(ds, st, c, a_hi, b_hi, Kp);
}

// The product kernel on prepared operand planes: A_hi, A_lo [M, Kp] from a_hi on, B^T_hi, B^T_lo [N, Kp] from b_hi on.
static int run_f32_planes(DeviceState *ds, cudaStream_t st, const GemmCall &c, float *a_hi, float *b_hi, long long Kp)
{
    const size_t a_plane = (size_t)c.M * Kp, b_plane = (size_t)c.N * Kp;
    int rc = BTM_OK;
    // The B box is one whole tile (bn rows), so the tile width is chosen here: 128 columns, or 64
    // when that leaves SMs without a tile.
    const long long t128 = (long long)((c.M + 127) / 128) * ((c.N + 127) / 128);
    const int bn = t128 < ds->sm_count ? 64 : 128;
    CUtensorMap tmA, tmB;
    rc = encode_tmap_3d(&tmA, BTM_F32, a_hi, (uint64_t)c.K, (uint64_t)c.M, 2, (uint64_t)Kp * 4, (uint64_t)a_plane * 4, 32, 128);
    if (rc) return rc;
    rc = encode_tmap_3d(&tmB, BTM_F32, b_hi, (uint64_t)c.K, (uint64_t)c.N, 2, (uint64_t)Kp * 4, (uint64_t)b_plane * 4, 32, bn);
    if (rc) return rc;
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.M = c.M;
    p.N = c.N;
    p.K = c.K;
    p.batch = 1;
    p.group_m = 8;
    p.ndst = 1;
    p.C[0] = c.C[0];
    p.ldc = c.ldc;
    p.c_vec_ok = (aligned16(c.C[0]) && (c.ldc * 4) % 16 == 0) ? 1 : 0;
    p.status = ds->status;
    fill_wait_params(&p);
    p.bias = c.bias;
    p.act = c.act;
    StoreMaps cm;
    rc = encode_store_maps(&cm, BTM_F32, p);
    if (rc) return rc;
    return launch_gemm_tc(BTM_F32, st, ds->sm_count, tmA, tmB, cm, p, bn);
}

static int check_gemm_args(int dtype, int M, int N, int K, const void *A, long long lda, const void *B, long long ldb,
                           const void *C, long long ldc)
{
    if (dtype != BTM_F16 && dtype != BTM_BF16 && dtype != BTM_F32)
        return set_error(BTM_ERR_UNSUPPORTED, "matmul: dtype %d is not supported (Float16, BFloat16, Float32 only)", dtype);
    if (M < 0 || N < 0 || K < 0) return set_error(BTM_ERR_INVALID, "matmul: negative dimension (M=%d N=%d K=%d)", M, N, K);
    if (M > 0 && N > 0 && !C) return set_error(BTM_ERR_INVALID, "matmul: null output pointer");
    if (M > 0 && K > 0 && !A) return set_error(BTM_ERR_INVALID, "matmul: null A pointer");
    if (K > 0 && N > 0 && !B) return set_error(BTM_ERR_INVALID, "matmul: null B pointer");
    if (lda < K || ldb < N || ldc < N)
        return set_error(BTM_ERR_INVALID, "matmul: leading dimension too small (lda=%lld ldb=%lld ldc=%lld for K=%d N=%d)", lda, ldb, ldc, K, N);
    const size_t es = es_of(dtype);
    if (((uintptr_t)A % es) || ((uintptr_t)B % es) || ((uintptr_t)C % es))
        return set_error(BTM_ERR_INVALID, "matmul: pointer not aligned to the element size");
    return BTM_OK;
}

} // namespace btm

using namespace btm;

extern "C" {

size_t btm_dtype_size(int dtype)
{
    switch (dtype) {
    case BTM_BF16: case BTM_F16: case BTM_I16: case BTM_U16: return 2;
    case BTM_F32: case BTM_I32: case BTM_U32: return 4;
    case BTM_F64: case BTM_I64: case BTM_U64: return 8;
    case BTM_I8: case BTM_U8: case BTM_INT4X2: return 1;
    default: return 0;
    }
}

int btm_version(void) { return 100; }

int btm_debug_set(const char *key, long long value)
{
    if (!key) return set_error(BTM_ERR_INVALID, "debug switch: null key");
    if (!strcmp(key, "wait_limit_cycles")) {
        if (value < 0) return set_error(BTM_ERR_INVALID, "debug switch wait_limit_cycles: negative value");
        g_dbg_wait_limit.store(value);
        return BTM_OK;
    }
    if (!strcmp(key, "skip_loads")) {
        g_dbg_skip_loads.store(value ? 1 : 0);
        return BTM_OK;
    }
    if (!strcmp(key, "bounds")) {
        g_dbg_bounds.store(value ? 1 : 0);
        return BTM_OK;
    }
    if (!strcmp(key, "bounds_shrink")) {
        if (value < 0) return set_error(BTM_ERR_INVALID, "debug switch bounds_shrink: negative value");
        g_dbg_bounds_shrink.store(value);
        return BTM_OK;
    }
    return set_error(BTM_ERR_INVALID, "debug switch: unknown key '%s'", key);
}

const char *btm_last_error_string(void) { return g_err; }

int btm_init(int device) { return device_state(device) ? BTM_OK : last_code(); }

int btm_check_device_status(int device, void *stream)
{
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    cudaStream_t st = (cudaStream_t)stream;
    int host = 0;
    int rc = check_cuda(cudaMemcpyAsync(&host, ds->status, sizeof(int), cudaMemcpyDeviceToHost, st), "status readback");
    if (rc) return rc;
    rc = check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize");
    if (rc) return rc;
    if (host != 0) {
        cudaMemsetAsync(ds->status, 0, sizeof(int), st);
        cudaStreamSynchronize(st);
        if (host == 201)
            return set_error(BTM_ERR_CUDA, "CUDA Error: a debug bounds check stopped a store outside the output (device status %d)", host);
        return set_error(BTM_ERR_TIMEOUT, "CUDA Error: a kernel wait ran out (device status %d)", host);
    }
    return BTM_OK;
}

static int gemm_entry(int device, void *stream, int dtype, int M, int N, int K, const void *A, int64_t lda, const void *B, int64_t ldb,
                      void *C, int64_t ldc, const void *bias, int act)
{
    int rc = check_gemm_args(dtype, M, N, K, A, lda, B, ldb, C, ldc);
    if (rc) return rc;
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    if (M == 0 || N == 0) return BTM_OK;
    cudaStream_t st = (cudaStream_t)stream;
    GemmCall c;
    memset(&c, 0, sizeof(c));
    c.dtype = dtype; c.batch = 1; c.M = M; c.N = N; c.K = K;
    c.A = A; c.B = B; c.lda = lda; c.ldb = ldb;
    c.C[0] = C; c.ndst = 1; c.ldc = ldc;
    c.bias = bias; c.act = act;
    if (dtype != BTM_F32) return run_16bit(ds, st, c);
    // fp32: the operand planes live in scratch that belongs to this call alone. It is taken from the library's pool
    // and given back in stream order on the caller's stream, so calls on other streams or threads never see it and
    // nothing is freed under work that is still queued.
    const size_t need = btm_gemm_f32_workspace_bytes(M, N, K);
    if (need == 0) return run_f32(ds, st, c, nullptr, 0);
    void *ws = nullptr;
    rc = check_cuda(cudaMallocFromPoolAsync(&ws, need, ds->pool, st), "cudaMallocFromPoolAsync(fp32 split scratch)");
    if (rc) return rc;
    rc = run_f32(ds, st, c, ws, need);
    const int rc_free = check_cuda(cudaFreeAsync(ws, st), "cudaFreeAsync(fp32 split scratch)");
    return rc ? rc : rc_free;
}

int btm_gemm(int device, void *stream, int dtype, int M, int N, int K, const void *A, int64_t lda, const void *B, int64_t ldb,
             void *C, int64_t ldc)
{
    return gemm_entry(device, stream, dtype, M, N, K, A, lda, B, ldb, C, ldc, nullptr, BTM_ACT_NONE);
}

int btm_gemm_bias_act(int device, void *stream, int dtype, int M, int N, int K, const void *A, int64_t lda, const void *B,
                      int64_t ldb, const void *bias, int act, void *C, int64_t ldc)
{
    if (act != BTM_ACT_NONE && act != BTM_ACT_RELU) return set_error(BTM_ERR_INVALID, "matmul: unknown activation %d", act);
    return gemm_entry(device, stream, dtype, M, N, K, A, lda, B, ldb, C, ldc, bias, act);
}

size_t btm_gemm_f32_workspace_bytes(int M, int N, int K)
{
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const size_t Kp = ((size_t)K + 3) & ~(size_t)3;
    return (2 * (size_t)M * Kp + 2 * (size_t)N * Kp) * sizeof(float);
}

int btm_gemm_f32_ws(int device, void *stream, int M, int N, int K, const void *A, int64_t lda, const void *B, int64_t ldb,
                    void *C, int64_t ldc, void *workspace, size_t workspace_bytes)
{
    int rc = check_gemm_args(BTM_F32, M, N, K, A, lda, B, ldb, C, ldc);
    if (rc) return rc;
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    if (M == 0 || N == 0) return BTM_OK;
    if (K > 0 && (!workspace || ((uintptr_t)workspace & 255)))
        return set_error(BTM_ERR_INVALID, "fp32 matmul: workspace must be non-null and 256-byte aligned");
    GemmCall c;
    memset(&c, 0, sizeof(c));
    c.dtype = BTM_F32; c.batch = 1; c.M = M; c.N = N; c.K = K;
    c.A = A; c.B = B; c.lda = lda; c.ldb = ldb;
    c.C[0] = C; c.ndst = 1; c.ldc = ldc;
    return run_f32(ds, (cudaStream_t)stream, c, workspace, workspace_bytes);
}

int btm_bmm(int device, void *stream, int dtype, int batch, int M, int N, int K, const void *A, int64_t strideA,
            const void *B, int64_t strideB, void *C, int64_t strideC)
{
    if (dtype != BTM_F16 && dtype != BTM_BF16)
        return set_error(BTM_ERR_UNSUPPORTED, "batched matmul: dtype %d is not supported (Float16, BFloat16 only)", dtype);
    if (batch < 0) return set_error(BTM_ERR_INVALID, "batched matmul: negative batch");
    int rc = check_gemm_args(dtype, M, N, K, A, K, B, N, C, N);
    if (rc) return rc;
    if (batch > 1 && (strideA < (int64_t)M * K || strideB < (int64_t)K * N || strideC < (int64_t)M * N))
        return set_error(BTM_ERR_INVALID, "batched matmul: batch stride smaller than one matrix");
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    if (batch == 0 || M == 0 || N == 0) return BTM_OK;
    GemmCall c;
    memset(&c, 0, sizeof(c));
    c.dtype = dtype; c.batch = batch; c.M = M; c.N = N; c.K = K;
    c.A = A; c.B = B; c.lda = K; c.ldb = N; c.strideA = strideA; c.strideB = strideB;
    c.C[0] = C; c.ndst = 1; c.ldc = N; c.strideC = strideC;
    return run_16bit(ds, (cudaStream_t)stream, c);
}

int btm_gemm_bt(int device, void *stream, int dtype, int M, int N, int K, const void *A, int64_t lda, const void *Bt, int64_t ldbt,
                void *C, int64_t ldc)
{
    if (dtype != BTM_F16 && dtype != BTM_BF16)
        return set_error(BTM_ERR_UNSUPPORTED, "matmul with transposed B: dtype %d is not supported (Float16, BFloat16 only)", dtype);
    int rc = check_gemm_args(dtype, M, N, K, A, lda, Bt, N /* checked below */, C, ldc);
    if (rc) return rc;
    if (ldbt < K) return set_error(BTM_ERR_INVALID, "matmul with transposed B: ldbt=%lld is smaller than K=%d", (long long)ldbt, K);
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    if (M == 0 || N == 0) return BTM_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t es = 2;
    if (K == 0 || !tma_ok(A, lda, 0, 1, es) || !tma_ok(Bt, ldbt, 0, 1, es))
        return set_error(BTM_ERR_UNSUPPORTED, "matmul with transposed B: operands must be 16-byte aligned with 16-byte row pitch and K > 0");
    const long long t256 = (long long)((M + 127) / 128) * ((N + 255) / 256);
    const int bn = t256 < ds->sm_count ? 128 : 256;
    CUtensorMap tmA, tmB;
    rc = encode_tmap_3d(&tmA, dtype, A, (uint64_t)K, (uint64_t)M, 1, (uint64_t)lda * es, (uint64_t)lda * es, 64, 128);
    if (rc) return rc;
    rc = encode_tmap_3d(&tmB, dtype, Bt, (uint64_t)K, (uint64_t)N, 1, (uint64_t)ldbt * es, (uint64_t)ldbt * es, 64, (uint32_t)bn);
    if (rc) return rc;
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.M = M; p.N = N; p.K = K; p.batch = 1; p.group_m = 8; p.ndst = 1;
    p.C[0] = C; p.ldc = ldc;
    p.c_vec_ok = (aligned16(C) && (ldc * (long long)es) % 16 == 0) ? 1 : 0;
    p.status = ds->status;
    fill_wait_params(&p);
    StoreMaps cm;
    rc = encode_store_maps(&cm, dtype, p);
    if (rc) return rc;
    return launch_gemm_tc_bt(dtype, st, ds->sm_count, tmA, tmB, cm, p, bn);
}

int btm_gemm_strided(int device, void *stream, int dtype, int M, int N, int K, const void *A, int64_t a_rs, int64_t a_cs, const void *B,
                     int64_t b_rs, int64_t b_cs, void *C, int64_t ldc)
{
    if (dtype != BTM_F16 && dtype != BTM_BF16 && dtype != BTM_F32)
        return set_error(BTM_ERR_UNSUPPORTED, "matmul: dtype %d is not supported (Float16, BFloat16, Float32 only)", dtype);
    if (M < 0 || N < 0 || K < 0) return set_error(BTM_ERR_INVALID, "matmul: negative dimension (M=%d N=%d K=%d)", M, N, K);
    if (a_rs < 0 || a_cs < 0 || b_rs < 0 || b_cs < 0) return set_error(BTM_ERR_INVALID, "matmul: negative strides are not supported");
    // Row-major operands are the plain product.
    if ((a_cs == 1 || K <= 1) && (b_cs == 1 || N <= 1))
        return btm_gemm(device, stream, dtype, M, N, K, A, M > 1 ? a_rs : std::max<int64_t>(K, 1), B, K > 1 ? b_rs : std::max<int64_t>(N, 1), C, ldc);
    if (M > 0 && N > 0 && !C) return set_error(BTM_ERR_INVALID, "matmul: null output pointer");
    if ((M > 0 && K > 0 && !A) || (K > 0 && N > 0 && !B)) return set_error(BTM_ERR_INVALID, "matmul: null operand pointer");
    if (ldc < N) return set_error(BTM_ERR_INVALID, "matmul: ldc=%lld is smaller than N=%d", (long long)ldc, N);
    const size_t es = es_of(dtype);
    if (((uintptr_t)A % es) || ((uintptr_t)B % es) || ((uintptr_t)C % es)) return set_error(BTM_ERR_INVALID, "matmul: pointer not aligned to the element size");
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    if (M == 0 || N == 0) return BTM_OK;
    cudaStream_t st = (cudaStream_t)stream;
    // Which operand is stored transposed (unit stride along the other index)? Anything else takes the general kernel.
    const bool a_row = a_cs == 1 || K <= 1, a_t = !a_row && (a_rs == 1 || M <= 1);
    const bool b_row = b_cs == 1 || N <= 1, b_t = !b_row && (b_rs == 1 || K <= 1);
    const bool unit = (a_row || a_t) && (b_row || b_t);
    if (dtype == BTM_F32 && unit && K > 0) {
        // The split pass rewrites both operands anyway: it reads them in whatever order they are stored.
        const long long Kp = (K + 3) & ~3LL;
        const size_t a_plane = (size_t)M * Kp, b_plane = (size_t)N * Kp, need = (2 * a_plane + 2 * b_plane) * sizeof(float);
        void *ws = nullptr;
        int rc = check_cuda(cudaMallocFromPoolAsync(&ws, need, ds->pool, st), "cudaMallocFromPoolAsync(fp32 split scratch)");
        if (rc) return rc;
        float *a_hi = (float *)ws, *a_lo = a_hi + a_plane, *b_hi = a_lo + a_plane, *b_lo = b_hi + b_plane;
        rc = a_t ? launch_split_tf32_transpose(st, (const float *)A, a_cs, K, M, a_hi, a_lo, Kp)
                 : launch_split_tf32(st, (const float *)A, a_rs, M, K, a_hi, a_lo, Kp);
        if (!rc)
            rc = b_t ? launch_split_tf32(st, (const float *)B, b_cs, N, K, b_hi, b_lo, Kp)
                     : launch_split_tf32_transpose(st, (const float *)B, b_rs, K, N, b_hi, b_lo, Kp);
        if (!rc) {
            GemmCall c;
            memset(&c, 0, sizeof(c));
            c.dtype = BTM_F32; c.batch = 1; c.M = M; c.N = N; c.K = K;
            c.C[0] = C; c.ndst = 1; c.ldc = ldc;
            rc = run_f32_planes(ds, st, c, a_hi, b_hi, Kp);
        }
        const int rc_free = check_cuda(cudaFreeAsync(ws, st), "cudaFreeAsync(fp32 split scratch)");
        return rc ? rc : rc_free;
    }
    if (dtype != BTM_F32 && unit && K > 0) {
        const long long lda = a_t ? a_cs : a_rs, ldb = b_t ? b_cs : b_rs;
        if (tma_ok(A, lda, 0, 1, es) && tma_ok(B, ldb, 0, 1, es)) {
            const long long t256 = (long long)((M + 127) / 128) * ((N + 255) / 256);
            const int bn = t256 < ds->sm_count ? 128 : 256;
            CUtensorMap tmA, tmB;
            int rc = a_t ? encode_tmap_3d(&tmA, dtype, A, (uint64_t)M, (uint64_t)K, 1, (uint64_t)lda * es, (uint64_t)lda * es, 64, 64)
                         : encode_tmap_3d(&tmA, dtype, A, (uint64_t)K, (uint64_t)M, 1, (uint64_t)lda * es, (uint64_t)lda * es, 64, 128);
            if (rc) return rc;
            rc = b_t ? encode_tmap_3d(&tmB, dtype, B, (uint64_t)K, (uint64_t)N, 1, (uint64_t)ldb * es, (uint64_t)ldb * es, 64, (uint32_t)bn)
                     : encode_tmap_3d(&tmB, dtype, B, (uint64_t)N, (uint64_t)K, 1, (uint64_t)ldb * es, (uint64_t)ldb * es, 64, 64);
            if (rc) return rc;
            GemmParams p;
            memset(&p, 0, sizeof(p));
            p.M = M; p.N = N; p.K = K; p.batch = 1; p.group_m = 8; p.ndst = 1;
            p.C[0] = C; p.ldc = ldc;
            p.c_vec_ok = (aligned16(C) && (ldc * (long long)es) % 16 == 0) ? 1 : 0;
            p.status = ds->status;
            fill_wait_params(&p);
            StoreMaps cm;
            rc = encode_store_maps(&cm, dtype, p);
            if (rc) return rc;
            return launch_gemm_tc_layout(dtype, st, ds->sm_count, tmA, tmB, cm, p, bn, a_t, b_t);
        }
    }
    // Arbitrary strides, unaligned transposed operands, K == 0: the general kernel, same arithmetic contract.
    return launch_gemm_simt(dtype, st, 1, M, N, K, A, a_rs, 0, B, b_rs, 0, C, ldc, 0, nullptr, 0, a_cs, b_cs);
}

int btm_gemm_nshard(int device, void *stream, int dtype, int M, int Nloc, int K, const void *A, int64_t lda,
                    const void *B_local, int64_t ldb, void *const *C_ranks, int64_t ldc, int rank, int nranks)
{
    if (dtype != BTM_F16 && dtype != BTM_BF16)
        return set_error(BTM_ERR_UNSUPPORTED, "sharded matmul: dtype %d is not supported (Float16, BFloat16 only)", dtype);
    if (nranks < 1 || nranks > kMaxDst || rank < 0 || rank >= nranks)
        return set_error(BTM_ERR_INVALID, "sharded matmul: rank %d of %d is out of range (at most %d ranks)", rank, nranks, kMaxDst);
    if (!C_ranks) return set_error(BTM_ERR_INVALID, "sharded matmul: null destination table");
    if (ldc < (int64_t)Nloc * nranks) return set_error(BTM_ERR_INVALID, "sharded matmul: ldc=%lld is smaller than nranks*Nloc", (long long)ldc);
    for (int r = 0; r < nranks; ++r)
        if (!C_ranks[r] && M > 0 && Nloc > 0) return set_error(BTM_ERR_INVALID, "sharded matmul: null C for rank %d", r);
    int rc = check_gemm_args(dtype, M, Nloc, K, A, lda, B_local, ldb, C_ranks[rank], ldc);
    if (rc) return rc;
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    if (M == 0 || Nloc == 0) return BTM_OK;
    GemmCall c;
    memset(&c, 0, sizeof(c));
    c.dtype = dtype; c.batch = 1; c.M = M; c.N = Nloc; c.K = K;
    c.A = A; c.B = B_local; c.lda = lda; c.ldb = ldb;
    // Local copy first, then the peers starting from the next rank so that the ranks do not
    // all write into the same peer at the same moment.
    c.C[0] = C_ranks[rank];
    for (int i = 1; i < nranks; ++i) c.C[i] = C_ranks[(rank + i) % nranks];
    c.ndst = nranks; c.ldc = ldc; c.col0 = (long long)rank * Nloc;
    return run_16bit(ds, (cudaStream_t)stream, c);
}

int btm_gemm_nshard_mc(int device, void *stream, int dtype, int M, int Nloc, int K, const void *A, int64_t lda, const void *B_local,
                       int64_t ldb, void *C_local, void *C_multicast, int64_t ldc, int rank, int nranks)
{
    if (dtype != BTM_F16 && dtype != BTM_BF16)
        return set_error(BTM_ERR_UNSUPPORTED, "sharded matmul: dtype %d is not supported (Float16, BFloat16 only)", dtype);
    if (nranks < 1 || nranks > kMaxDst || rank < 0 || rank >= nranks)
        return set_error(BTM_ERR_INVALID, "sharded matmul: rank %d of %d is out of range (at most %d ranks)", rank, nranks, kMaxDst);
    if (!C_multicast || !C_local) return set_error(BTM_ERR_INVALID, "sharded matmul: null output mapping");
    if (ldc < (int64_t)Nloc * nranks) return set_error(BTM_ERR_INVALID, "sharded matmul: ldc=%lld is smaller than nranks*Nloc", (long long)ldc);
    int rc = check_gemm_args(dtype, M, Nloc, K, A, lda, B_local, ldb, C_local, ldc);
    if (rc) return rc;
    // The multimem stores are 16 bytes wide and unpredicated inside a chunk of 8 columns, and the operands must be
    // addressable by the tensor-core kernels (there is no general-kernel form of the multicast epilogue).
    if (K <= 0 || (Nloc % 8) || (ldc % 8) || (((uintptr_t)C_multicast | (uintptr_t)C_local) & 15) || !tma_ok(A, lda, 0, 1, 2) || !tma_ok(B_local, ldb, 0, 1, 2))
        return set_error(BTM_ERR_UNSUPPORTED, "sharded matmul over multicast memory: needs K > 0, Nloc and ldc multiples of 8, 16-byte aligned operands");
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    if (M == 0 || Nloc == 0) return BTM_OK;
    GemmCall c;
    memset(&c, 0, sizeof(c));
    c.dtype = dtype; c.batch = 1; c.M = M; c.N = Nloc; c.K = K;
    c.A = A; c.B = B_local; c.lda = lda; c.ldb = ldb;
    c.C[0] = C_local; c.ndst = 1; c.mc = C_multicast;
    c.ldc = ldc; c.col0 = (long long)rank * Nloc;
    return run_16bit(ds, (cudaStream_t)stream, c);
}

int btm_int4_matmul(int device, void *stream, int M, int N, int K, int group, const void *act_f16, const void *w_packed,
                    const void *scales_f16, void *out_f16)
{
    if (M < 0 || N < 0 || K < 0) return set_error(BTM_ERR_INVALID, "int4 matmul: negative dimension");
    if (group <= 0 || K % 2 || (K % group) != 0) return set_error(BTM_ERR_INVALID, "int4 matmul: K=%d must be even and a multiple of group=%d", K, group);
    if (M > 0 && N > 0 && (!out_f16 || (K > 0 && (!act_f16 || !w_packed || !scales_f16))))
        return set_error(BTM_ERR_INVALID, "int4 matmul: null pointer");
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    // More than 8 activation rows: dequantise into shared memory and multiply on tcgen05 (weights read
    // from HBM once for up to 128 rows). BTM_FORCE_INT4=mma keeps the mma.sync kernels (tests cover both).
    const char *force = getenv("BTM_FORCE_INT4");
    const bool tc_ok = M > 8 && N > 0 && K >= 128 && K % 128 == 0 && group % 64 == 0 &&
                       (((uintptr_t)act_f16 | (uintptr_t)w_packed) & 15) == 0 && (((uintptr_t)scales_f16 | (uintptr_t)out_f16) & 1) == 0 &&
                       !(force && !strcmp(force, "mma"));
    // Many activation rows (prefill-sized M): the tcgen05 int4 kernel re-reads and re-unpacks the weights for every 128
    // rows, so from a few hundred rows on it is cheaper to write the dequantised weights (the btm_int4_dequant values,
    // which are what that kernel multiplies by as well) once into stream-ordered scratch and run one dense product
    // with them as the K-major operand. BTM_INT4_LARGE_M moves the threshold (tests run both sides of it).
    int large_m = 640; // measured crossover at N = 11008, K = 4096: 512 rows 73 us per pass against 90 us, 768 rows 110 against 92 us
    if (const char *lm = getenv("BTM_INT4_LARGE_M")) large_m = std::max(9, atoi(lm));
    if (tc_ok && M >= large_m && (((uintptr_t)out_f16) & 15) == 0 && N % 8 == 0) {
        cudaStream_t st = (cudaStream_t)stream;
        void *dq = nullptr;
        int rc = check_cuda(cudaMallocFromPoolAsync(&dq, (size_t)N * K * 2, ds->pool, st), "cudaMallocFromPoolAsync(int4 dequantised weights)");
        if (rc) return rc;
        rc = launch_int4_dequant(st, N, K, group, w_packed, scales_f16, dq);
        if (!rc) rc = btm_gemm_bt(device, stream, BTM_F16, M, N, K, act_f16, K, dq, K, out_f16, N);
        const int rc_free = check_cuda(cudaFreeAsync(dq, st), "cudaFreeAsync(int4 dequantised weights)");
        if (rc != BTM_ERR_UNSUPPORTED) return rc ? rc : rc_free;
    }
    if (tc_ok) {
        int rc = launch_int4_gemm_tc((cudaStream_t)stream, M, N, K, group, act_f16, w_packed, scales_f16, out_f16, ds->status, ds->sm_count);
        if (rc != BTM_ERR_UNSUPPORTED) return rc; // unsupported: scales too many for shared memory, nothing launched
    }
    return launch_int4_gemv((cudaStream_t)stream, ds->sm_count, M, N, K, group, act_f16, w_packed, scales_f16, out_f16, ds->status);
}

int btm_int4_dequant(int device, void *stream, int N, int K, int group, const void *w_packed, const void *scales_f16,
                     void *out_f16)
{
    if (N < 0 || K < 0) return set_error(BTM_ERR_INVALID, "int4 dequant: negative dimension");
    if (group <= 0 || K % 2 || (K % group) != 0) return set_error(BTM_ERR_INVALID, "int4 dequant: K=%d must be even and a multiple of group=%d", K, group);
    if ((long long)N * K > 0 && (!w_packed || !scales_f16 || !out_f16)) return set_error(BTM_ERR_INVALID, "int4 dequant: null pointer");
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    return launch_int4_dequant((cudaStream_t)stream, N, K, group, w_packed, scales_f16, out_f16);
}

int btm_int4_unpack(int device, void *stream, int N, int K, const void *w_packed, void *out_i8)
{
    if (N < 0 || K < 0 || K % 2) return set_error(BTM_ERR_INVALID, "int4 unpack: K=%d must be even and dimensions non-negative", K);
    if ((long long)N * K > 0 && (!w_packed || !out_i8)) return set_error(BTM_ERR_INVALID, "int4 unpack: null pointer");
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    return launch_int4_unpack((cudaStream_t)stream, N, K, w_packed, out_i8);
}

int btm_convert(int device, void *stream, int src_dtype, int dst_dtype, int64_t n, const void *src, void *dst)
{
    if (n < 0) return set_error(BTM_ERR_INVALID, "convert: negative element count");
    if (n > 0 && (!src || !dst)) return set_error(BTM_ERR_INVALID, "convert: null pointer");
    if (src_dtype == dst_dtype) return set_error(BTM_ERR_INVALID, "convert: source and destination dtype are the same");
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    return launch_convert((cudaStream_t)stream, src_dtype, dst_dtype, n, src, dst);
}

int btm_int4_quantize(int device, void *stream, int N, int K, int group, const void *w_f16, void *out_packed, void *out_scales_f16)
{
    if (N < 0 || K < 0) return set_error(BTM_ERR_INVALID, "int4 quantise: negative dimension");
    if (group <= 0 || group % 2 || (K % group) != 0) return set_error(BTM_ERR_INVALID, "int4 quantise: K=%d must be a multiple of the even group=%d", K, group);
    if ((long long)N * K > 0 && (!w_f16 || !out_packed || !out_scales_f16)) return set_error(BTM_ERR_INVALID, "int4 quantise: null pointer");
    DeviceState *ds = device_state(device);
    if (!ds) return last_code();
    return launch_int4_quantize((cudaStream_t)stream, N, K, group, w_f16, out_packed, out_scales_f16);
}

int btm_replicate_rows(int device, void *stream, void *const *bufs, int rank, int nranks, size_t offset_bytes, size_t bytes)
{
    if (nranks < 1 || nranks > kMaxDst || rank < 0 || rank >= nranks)
        return set_error(BTM_ERR_INVALID, "replicate: rank %d of %d is out of range (at most %d ranks)", rank, nranks, kMaxDst);
    if (!bufs) return set_error(BTM_ERR_INVALID, "replicate: null buffer table");
    for (int r = 0; r < nranks; ++r)
        if (!bufs[r]) return set_error(BTM_ERR_INVALID, "replicate: null buffer for rank %d", r);
    if (!device_state(device)) return last_code();
    if (bytes == 0) return BTM_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const char *src = (const char *)bufs[rank] + offset_bytes;
    // One copy per peer, starting with the next rank so that the ranks do not all write into the same peer first.
    for (int i = 1; i < nranks; ++i) {
        char *dst = (char *)bufs[(rank + i) % nranks] + offset_bytes;
        int rc = check_cuda(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st), "cudaMemcpyAsync(peer)");
        if (rc) return rc;
    }
    return BTM_OK;
}

int btm_ipc_alloc(int device, size_t bytes, void **ptr, unsigned char handle[64])
{
    if (!ptr || !handle || bytes == 0) return set_error(BTM_ERR_INVALID, "ipc alloc: bad arguments");
    if (!device_state(device)) return last_code();
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    int rc = check_cuda(cudaMalloc(ptr, bytes), "cudaMalloc(ipc)");
    if (rc) return rc;
    cudaIpcMemHandle_t h;
    rc = check_cuda(cudaIpcGetMemHandle(&h, *ptr), "cudaIpcGetMemHandle");
    if (rc) {
        cudaFree(*ptr);
        *ptr = nullptr;
        return rc;
    }
    memcpy(handle, &h, 64);
    return BTM_OK;
}

int btm_ipc_open(int device, const unsigned char handle[64], void **ptr)
{
    if (!ptr || !handle) return set_error(BTM_ERR_INVALID, "ipc open: bad arguments");
    if (!device_state(device)) return last_code();
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    return check_cuda(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
}

int btm_ipc_close(int device, void *ptr)
{
    if (!device_state(device)) return last_code();
    return check_cuda(cudaIpcCloseMemHandle(ptr), "cudaIpcCloseMemHandle");
}

int btm_ipc_free(int device, void *ptr)
{
    if (!device_state(device)) return last_code();
    return check_cuda(cudaFree(ptr), "cudaFree(ipc)");
}

} // extern "C"
