// btm_gemm_f32_static: the fp32 (3xTF32) matmul for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a product: a
// thread-pool worker that runs while another thread holds the allocator, code that has handed
// all device memory to its own pool at start-up, or a service whose memory budget is fixed once
// and audited. The ordinary fp32 entry point keeps a per-device scratch buffer and grows it with
// cudaMalloc when a larger shape arrives, so it is not usable there. This variant runs the same
// kernels with the scratch (the hi/lo operand planes) in a fixed array that is part of the
// library image: nothing is allocated or freed, on any call.
//
// The price: the array has a fixed size (BTM_STATIC_SCRATCH_BYTES, 64 MiB, which every GPU that
// loads the library holds until the process exits), larger products are refused, and every call
// on a device shares the one array — two calls whose kernels overlap on the GPU (different
// streams, or different host threads without ordering) race on it and corrupt each other's
// operands. Order such calls on one stream.
#include <cstring>
#include <mutex>

#include "btm_internal.h"

namespace {

constexpr size_t kStaticScratchBytes = 64ull << 20;

// File-scope device storage. In host code these names are only stand-ins for the symbols: the
// device addresses are obtained once per device with cudaGetSymbolAddress (below) and it is those
// addresses that reach the kernels.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ int g_static_status; // bounded-wait report of this entry point's kernels (starts 0)

struct StaticDeviceState {
    bool ready;
    void *scratch; // device address of g_static_scratch on this device
    int *status;   // device address of g_static_status on this device
    int sm_count;
};

constexpr int kMaxDevices = 64;
StaticDeviceState g_state[kMaxDevices];
std::mutex g_mu;

// One-time set-up for `device`, which the caller has already made current. No allocation:
// symbol lookups and kernel attribute changes only.
StaticDeviceState *setup(int device, int *code)
{
    std::lock_guard<std::mutex> lock(g_mu);
    StaticDeviceState *s = &g_state[device];
    *code = BTM_ERR_CUDA;
    if (s->ready) return s;
    cudaDeviceProp prop;
    if (btm::check_cuda(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties")) return nullptr;
    if (prop.major != 10) {
        *code = btm::set_error(BTM_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major,
                               prop.minor);
        return nullptr;
    }
    void *scratch = nullptr, *status = nullptr;
    if (btm::check_cuda(cudaGetSymbolAddress(&scratch, g_static_scratch), "cudaGetSymbolAddress(static scratch)")) return nullptr;
    if (btm::check_cuda(cudaGetSymbolAddress(&status, g_static_status), "cudaGetSymbolAddress(static status)")) return nullptr;
    if (btm::configure_gemm_tc_kernels()) return nullptr;
    s->scratch = scratch;
    s->status = (int *)status;
    s->sm_count = prop.multiProcessorCount;
    s->ready = true;
    return s;
}

} // namespace

extern "C" int btm_gemm_f32_static(int device, void *stream, int M, int N, int K, const void *A, int64_t lda, const void *B,
                                   int64_t ldb, void *C, int64_t ldc)
{
    using namespace btm;
    if (M < 0 || N < 0 || K < 0) return set_error(BTM_ERR_INVALID, "matmul: negative dimension (M=%d N=%d K=%d)", M, N, K);
    if (M == 0 || N == 0) return BTM_OK;
    if (!C || (K > 0 && (!A || !B))) return set_error(BTM_ERR_INVALID, "matmul: null pointer");
    if (lda < K || ldb < N || ldc < N)
        return set_error(BTM_ERR_INVALID, "matmul: leading dimension too small (lda=%lld ldb=%lld ldc=%lld for K=%d N=%d)",
                         (long long)lda, (long long)ldb, (long long)ldc, K, N);
    if (((uintptr_t)A & 3) || ((uintptr_t)B & 3) || ((uintptr_t)C & 3))
        return set_error(BTM_ERR_INVALID, "matmul: pointer not aligned to the element size");
    const long long Kp = ((long long)K + 3) & ~3LL;
    const size_t a_plane = (size_t)M * Kp, b_plane = (size_t)N * Kp;
    const size_t need = (2 * a_plane + 2 * b_plane) * sizeof(float);
    if (need > kStaticScratchBytes)
        return set_error(BTM_ERR_UNSUPPORTED,
                         "fp32 matmul without allocation: M=%d N=%d K=%d needs %zu bytes of scratch, the built-in array holds %zu "
                         "((M+N)*roundup(K,4)*8 must not exceed it); use btm_gemm or btm_gemm_f32_ws for larger products",
                         M, N, K, need, kStaticScratchBytes);
    if (device < 0 || device >= kMaxDevices) return set_error(BTM_ERR_INVALID, "Invalid GPU ID %d", device);
    int count = 0;
    int rc = check_cuda(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
    if (rc) return rc;
    if (device >= count) return set_error(BTM_ERR_INVALID, "Invalid GPU ID %d (device count %d)", device, count);
    rc = check_cuda(cudaSetDevice(device), "cudaSetDevice");
    if (rc) return rc;
    int setup_code = BTM_ERR_CUDA;
    StaticDeviceState *s = setup(device, &setup_code);
    if (!s) return setup_code;
    cudaStream_t st = (cudaStream_t)stream;

    // A wait that ran out in an earlier call of this entry point left a code in the private status word. It is
    // looked at only when `stream` is not being captured and has nothing queued: the read then goes through
    // `stream` itself (no other stream is touched) and returns at once.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    rc = check_cuda(cudaStreamIsCapturing(st, &cap), "cudaStreamIsCapturing");
    if (rc) return rc;
    if (cap == cudaStreamCaptureStatusNone) {
        const cudaError_t q = cudaStreamQuery(st);
        if (q == cudaSuccess) {
            int code = 0;
            rc = check_cuda(cudaMemcpyAsync(&code, s->status, sizeof(int), cudaMemcpyDeviceToHost, st), "status readback");
            if (rc) return rc;
            rc = check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize");
            if (rc) return rc;
            if (code != 0) {
                rc = check_cuda(cudaMemsetAsync(s->status, 0, sizeof(int), st), "status clear");
                if (rc) return rc;
                return set_error(BTM_ERR_TIMEOUT, "CUDA Error: a kernel wait ran out in an earlier call (device status %d)", code);
            }
        } else if (q == cudaErrorNotReady) {
            (void)cudaGetLastError(); // work is queued: expected, and it must not stick as the thread's last error
        } else {
            return check_cuda(q, "cudaStreamQuery");
        }
    }

    if (K == 0) return launch_gemm_simt(BTM_F32, st, 1, M, N, 0, A, lda, 0, B, ldb, 0, C, ldc, 0);

    // Planes in the static array: A_hi, A_lo [M,Kp], then B^T_hi, B^T_lo [N,Kp]. The split passes
    // overwrite every element that the product reads, so stale contents of an earlier call are harmless.
    float *a_hi = (float *)s->scratch, *a_lo = a_hi + a_plane, *b_hi = a_lo + a_plane, *b_lo = b_hi + b_plane;
    rc = launch_split_tf32(st, (const float *)A, lda, M, K, a_hi, a_lo, Kp);
    if (rc) return rc;
    rc = launch_split_tf32_transpose(st, (const float *)B, ldb, K, N, b_hi, b_lo, Kp);
    if (rc) return rc;
    const long long t128 = (long long)((M + 127) / 128) * ((N + 127) / 128);
    const int bn = t128 < s->sm_count ? 64 : 128;
    CUtensorMap tmA, tmB;
    rc = encode_tmap_3d(&tmA, BTM_F32, a_hi, (uint64_t)K, (uint64_t)M, 2, (uint64_t)Kp * 4, (uint64_t)a_plane * 4, 32, 128);
    if (rc) return rc;
    rc = encode_tmap_3d(&tmB, BTM_F32, b_hi, (uint64_t)K, (uint64_t)N, 2, (uint64_t)Kp * 4, (uint64_t)b_plane * 4, 32, (uint32_t)bn);
    if (rc) return rc;
    GemmParams p;
    memset(&p, 0, sizeof(p));
    p.M = M;
    p.N = N;
    p.K = K;
    p.batch = 1;
    p.group_m = 8;
    p.ndst = 1;
    p.C[0] = C;
    p.ldc = ldc;
    p.c_vec_ok = ((((uintptr_t)C) & 15) == 0 && (ldc * 4) % 16 == 0) ? 1 : 0; // same store path as btm_gemm
    p.status = s->status;
    fill_wait_params(&p);
    StoreMaps cm;
    rc = encode_store_maps(&cm, BTM_F32, p);
    if (rc) return rc;
    return launch_gemm_tc(BTM_F32, st, s->sm_count, tmA, tmB, cm, p, bn);
}
