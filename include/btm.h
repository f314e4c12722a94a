/*
 * btm.h — C ABI of libbtm.so, the sm_100a matmul subsystem that sits behind BeanTensor's
 * GPU operator boundary (namespace BeanTensor::Tensors::detail, Tensor/TensorOps.h:15-65).
 *
 * The reference declares its GPU operators as free functions taking Tensor& and running
 * on a thread-pool worker (Tensor/TensorOps.cu:89-208). It has no matmul of its own
 * (Ops/Algebra/MatMul/MatMul.h:1-8 is an empty include guard), so each entry point below
 * names the reference interface it extends or stands in for. A BeanTensor maintainer
 * binds these from a `detail::matmul_gpu(const Tensor&, const Tensor&, Tensor&)` style
 * function; beantensor_b200/host/MatMulOps.h is that binding.
 *
 * Conventions shared by every call
 *   - plain pointers and sizes only; all matrices are row-major with leading dimensions
 *     in ELEMENTS (Tensor/Tensor.cpp:157-162);
 *   - `dtype` is the reference's DType ordinal (Tensor/Dtypes.h:57-70);
 *   - `device` is the CUDA ordinal (Tensor::gpu_id, Tensor/Tensor.h:191); the call makes
 *     it current on the calling thread itself, because the reference's pool threads set
 *     it inconsistently (Tensor/TensorOps.cu:232-259 does, :89-208 does not);
 *   - `stream` is a cudaStream_t passed as void* (NULL = the null stream, which is what
 *     the reference always uses, Tensor/Tensor.h:187); work is enqueued, not awaited;
 *   - the caller owns every buffer; outputs are pre-allocated (ops never reallocate
 *     Tensor::data, cf. Tensor/TensorOps.cu:89-208);
 *   - the return value is a btm_status; a C ABI cannot throw, so the C++ binding maps the
 *     status back to the reference's exception types (Errors/Logic.h:13-38);
 *   - calls are re-entrant and may come from any thread (Helper/Threads/CPUThreading.h:37-56); two calls share
 *     nothing but read-only per-device state, unless an entry point below says otherwise.
 * There is no CPU fallback: without a usable sm_100 device every compute call fails with
 * BTM_ERR_CUDA or BTM_ERR_UNSUPPORTED.
 */
#ifndef BTM_H
#define BTM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes. Mapping in the C++ binding: INVALID -> std::invalid_argument
 * (Tensor/TensorOps.cu:241,269), UNSUPPORTED -> ErrorHandling::NotImplemented
 * (Errors/Logic.h:13-17), OOM -> ErrorHandling::OutOfMemory (Errors/Logic.h:22-25),
 * CUDA/NCCL/TIMEOUT -> std::runtime_error("CUDA Error: ...") (Errors/Logic.h:50-59). */
typedef enum btm_status {
    BTM_OK = 0,
    BTM_ERR_INVALID = 1,
    BTM_ERR_UNSUPPORTED = 2,
    BTM_ERR_OOM = 3,
    BTM_ERR_CUDA = 4,
    BTM_ERR_NCCL = 5,
    BTM_ERR_TIMEOUT = 6
} btm_status;

/* DType ordinals: identical to enum class DType, Tensor/Dtypes.h:57-70. INT4X2 is
 * appended (the reference has no sub-byte type) so ordinals 0..11 keep their meaning:
 * one byte holds two signed 4-bit values, even k in bits 0-3, odd k in bits 4-7. */
typedef enum btm_dtype {
    BTM_BF16 = 0,
    BTM_F16 = 1,
    BTM_F32 = 2,
    BTM_F64 = 3,
    BTM_I64 = 4,
    BTM_I32 = 5,
    BTM_I16 = 6,
    BTM_I8 = 7,
    BTM_U64 = 8,
    BTM_U32 = 9,
    BTM_U16 = 10,
    BTM_U8 = 11,
    BTM_INT4X2 = 12
} btm_dtype;

/* POD mirror of the fields of class Tensor that the path reads (Tensor/Tensor.h:173-201):
 * shape and strides in elements, at most 8 dims, offset in elements. */
typedef struct btm_tensor_view {
    void *data;
    int32_t dtype;  /* btm_dtype */
    int32_t device; /* 0 = CPU, 1 = GPU (enum class Device, Tensor/Tensor.h:34-37) */
    int32_t gpu_id;
    int32_t ndim;
    uint64_t shape[8];
    uint64_t strides[8];
    uint64_t offset;
} btm_tensor_view;

/* Element size in bytes of a dtype ordinal (dtype_size, Tensor/Dtypes.h:75-92);
 * BTM_INT4X2 reports 1 (one byte = two elements); unknown ordinals report 0. */
size_t btm_dtype_size(int dtype);

/* Library version, major*10000 + minor*100 + patch. */
int btm_version(void);

/* Text of the last error raised on the calling thread (never NULL). Plays the role of
 * the what() string of the exceptions the reference throws (Errors/Logic.h:13-59). */
const char *btm_last_error_string(void);

/* Test hooks, no counterpart in the reference. Process-wide switches that make the bounded waits inside the
 * matmul kernels observable without any fault: "wait_limit_cycles" (SM cycles after which a kernel wait gives
 * up; 0 restores the default of about one second) and "skip_loads" (non-zero: the producer warps of the dense
 * matmul kernels issue no loads, so the consumers' waits run out, the kernel unwinds, returns, and the next
 * btm_check_device_status reports BTM_ERR_TIMEOUT); "bounds" (non-zero: every store address that a matmul epilogue
 * computes by hand is compared with the extent of C first, a store that would leave it is skipped and reported by
 * btm_check_device_status as BTM_ERR_CUDA; also switched on by the environment variable BTM_DEBUG_BOUNDS=1, read once)
 * and "bounds_shrink" (pretend C is that many elements shorter, so that a test can watch the check fire without any
 * access outside memory). Unknown keys return BTM_ERR_INVALID. */
int btm_debug_set(const char *key, long long value);

/* Prepare `device`: checks that it is an sm_100 part, creates the per-device state
 * (status word, kernel attributes). Every compute call does this lazily; call it up front
 * to keep the first timed call clean. Stands where the reference's workers do their
 * device checks (Tensor/TensorOps.cu:236-247). */
int btm_init(int device);

/* Reads and clears the device-side status word that kernels set when one of their
 * bounded waits ran out. Synchronises `stream`. Returns BTM_OK or BTM_ERR_TIMEOUT. */
int btm_check_device_status(int device, void *stream);

/* Dense matmul C[M,N] = A[M,K] . B[K,N], the op that Ops/Algebra/MatMul/MatMul.h:1-8
 * leaves empty; to be called from a detail::matmul_gpu() declared beside the functions of
 * Tensor/TensorOps.h:18-63.
 *   dtype BTM_F16 / BTM_BF16: fp32 accumulation on the tensor cores, output rounded to
 *   nearest even into the same 16-bit type (as Tensor/TensorOps.cu:72 rounds).
 *   dtype BTM_F32: three-term TF32 split (hi.hi + hi.lo + lo.hi) with fp32 accumulation;
 *   needs (M + N) * roundup(K,4) * 8 bytes of scratch. Every call takes its own block from a memory
 *   pool that the library keeps per device and returns it in stream order on `stream`
 *   (cudaMallocFromPoolAsync / cudaFreeAsync), so concurrent calls on other streams or threads never
 *   share scratch; freed blocks stay in the pool, and only the first call of a larger shape reaches
 *   the driver. Infinite inputs give infinite (not NaN) outputs, as a plain fp32 product would.
 * lda >= K, ldb >= N, ldc >= N, in elements. Any M, N, K >= 0; shapes or pointers that
 * the tensor-core path cannot address (row pitch or base not 16-byte aligned) run on a
 * general CUDA-core kernel with the same arithmetic contract. */
int btm_gemm(int device, void *stream, int dtype, int M, int N, int K, const void *A, int64_t lda, const void *B,
             int64_t ldb, void *C, int64_t ldc);

/* Fused epilogue: C[M,N] = act(A[M,K] . B[K,N] + bias[N]), where the bias (one value per output column, same
 * dtype as C, or NULL for none) is added to the fp32 accumulator and the activation applied before the single
 * rounding to the output type. This is the fusion of the product with the reference's element-wise Add
 * (Ops/Elementwise/Add/Add.h:28, broadcast of a row vector) and Relu (Ops/Elementwise/Relu/Relu.h, an empty
 * include guard) into the kernel that produces C, so C is written once. Everything else as btm_gemm. */
enum btm_activation { BTM_ACT_NONE = 0, BTM_ACT_RELU = 1 };
int btm_gemm_bias_act(int device, void *stream, int dtype, int M, int N, int K, const void *A, int64_t lda, const void *B,
                      int64_t ldb, const void *bias, int act, void *C, int64_t ldc);

/* C[M,N] = A[M,K] . Bt[N,K]^T: the same product with B supplied transposed (row-major [N,K], so both
 * operands are K-contiguous). This is the copy-free form of matmul(a, transpose(b)); the reference's
 * Ops/Algebra/Transpose is an empty stub (Ops/Algebra/Transpose/Transpose.h), so a BeanTensor
 * caller would otherwise have to materialise the transpose. BTM_F16 / BTM_BF16, tensor-core path only:
 * bases and row pitches must be multiples of 16 bytes and K > 0, else BTM_ERR_UNSUPPORTED. */
int btm_gemm_bt(int device, void *stream, int dtype, int M, int N, int K, const void *A, int64_t lda, const void *Bt,
                int64_t ldbt, void *C, int64_t ldc);

/* The same product for operands that are not row-major: A[m,k] lies at A + m*a_rs + k*a_cs and B[k,n] at
 * B + k*b_rs + n*b_cs (element strides, as in Tensor::strides, Tensor/Tensor.h:173-195); C stays row-major with ldc.
 * This is what lets matmul(transpose(a), b), matmul(a, transpose(b)) and products of strided views run without a copy;
 * the reference's Ops/Algebra/Transpose is an empty stub (Ops/Algebra/Transpose/Transpose.h), so its callers would
 * have to materialise such operands first. An operand with unit stride along either index takes the tensor-core
 * kernels (a transposed 16-bit operand is read as an MN-major tensor-core operand through its tensor map; the fp32
 * split pass reads its operands in whatever order they are stored), provided bases and pitches are multiples of
 * 16 bytes; anything else takes the general CUDA-core kernel with the same arithmetic contract. Strides >= 0. */
int btm_gemm_strided(int device, void *stream, int dtype, int M, int N, int K, const void *A, int64_t a_rs, int64_t a_cs,
                     const void *B, int64_t b_rs, int64_t b_cs, void *C, int64_t ldc);

/* Same product for BTM_F32 with caller-owned scratch instead of the library's:
 * `workspace` is device memory of at least btm_gemm_f32_workspace_bytes(M,N,K) bytes,
 * 256-byte aligned. Nothing is allocated. */
size_t btm_gemm_f32_workspace_bytes(int M, int N, int K);
int btm_gemm_f32_ws(int device, void *stream, int M, int N, int K, const void *A, int64_t lda, const void *B,
                    int64_t ldb, void *C, int64_t ldc, void *workspace, size_t workspace_bytes);

/* fp32 matmul for callers that cannot allocate. No counterpart in the reference (it has no matmul,
 * and its operators allocate freely, e.g. Tensor/TensorOps.cu:248,329-333).
 * Who needs it: a worker that runs while another thread owns the CUDA allocator, a host that gave
 * all device memory to its own pool at start-up, a service with a fixed, audited memory budget. For
 * them btm_gemm(BTM_F32) is unusable because it grows its scratch with cudaMalloc. This call does the
 * same three-term TF32 product with the operand planes in a fixed array inside the library image:
 * it never calls cudaMalloc, cudaFree or any allocating routine.
 * Limits and rules:
 *   - (M + N) * roundup(K,4) * 8 bytes must not exceed BTM_STATIC_SCRATCH_BYTES (64 MiB, e.g. up to
 *     2048^3); larger products return BTM_ERR_UNSUPPORTED with a message that says so. Every GPU
 *     that loads the library holds those 64 MiB until the process exits.
 *   - all calls on a device share the one array: calls whose kernels can overlap on the GPU
 *     (different streams, unordered host threads) race on it. Order them on one stream.
 *   - the first call on a device looks up the array's device address (once per device); make that
 *     first call before starting any stream capture.
 *   - a kernel wait that ran out is reported by a later call of this function on the same device
 *     (BTM_ERR_TIMEOUT). That check reads one word back through `stream` and is made only when
 *     `stream` is idle and not being captured; no other stream is touched. */
#define BTM_STATIC_SCRATCH_BYTES (64ull << 20)
int btm_gemm_f32_static(int device, void *stream, int M, int N, int K, const void *A, int64_t lda, const void *B,
                        int64_t ldb, void *C, int64_t ldc);

/* Batched matmul: `batch` independent products C[b] = A[b] . B[b] with element strides
 * between consecutive matrices; each matrix is row-major and dense (lda=K, ldb=N, ldc=N).
 * The reference has no such op (not even a stub); it extends Ops/Algebra/MatMul the same
 * way. dtype BTM_F16 or BTM_BF16. One persistent launch walks all (batch, tile) pairs. */
int btm_bmm(int device, void *stream, int dtype, int batch, int M, int N, int K, const void *A, int64_t strideA,
            const void *B, int64_t strideB, void *C, int64_t strideC);

/* int4 weight-only matmul: out[M,N] (fp16) = act[M,K] (fp16) . dequant(W)[N,K]^T with
 * W packed two nibbles per byte along K ([N, K/2] bytes) and one fp16 scale per `group`
 * consecutive k ([N, K/group]). The dtype is this build's addition to Tensor/Dtypes.h:57-70.
 * Arithmetic: fp32 accumulation of act*w inside a group, times the scale, summed over
 * groups, rounded to nearest even (for M > 8 the weights are first rounded to fp16 as
 * btm_int4_dequant defines them and the product accumulates in fp32; from 640 rows on those
 * fp16 weights are written once into stream-ordered scratch of N*K*2 bytes from the library's
 * per-device pool and multiplied by the dense tensor-core kernel, instead of being unpacked again
 * for every 128 rows). K % group == 0, group % 32 == 0, K % 32 == 0.
 * Ordering: the products use programmatic dependent launch. If the preceding kernel on the
 * stream is another int4 product of this library, this one may read w_packed and scales_f16 while
 * that kernel is still running (act_f16 is read and out_f16 written only after it has completed);
 * w_packed and scales_f16 must therefore not be the output of an immediately preceding int4 product. */
int btm_int4_matmul(int device, void *stream, int M, int N, int K, int group, const void *act_f16,
                    const void *w_packed, const void *scales_f16, void *out_f16);

/* Bit-exact dequantisation of the packed weights to fp16 [N,K]:
 * out[n,k] = f16_rne(float(W[n,k]) * float(S[n,k/group])). Plays the role of a
 * convert_gpu() case (Tensor/TensorOps.cu:315-365) for the appended dtype. */
int btm_int4_dequant(int device, void *stream, int N, int K, int group, const void *w_packed,
                     const void *scales_f16, void *out_f16);

/* Group quantiser, the producer of the packed format: for every row n and group g of `group` consecutive k,
 * S[n,g] = f16_rne(max|w| / 7) (1 when the group is all zero) and
 * W[n,k] = clamp(rint(float(w[n,k]) / float(S[n,g])), -8, 7) with round-half-to-even, packed two per byte.
 * fp16 in, bytes [N,K/2] and fp16 scales [N,K/group] out. The reference has no quantised type; this is
 * the convert_gpu() case (Tensor/TensorOps.cu:315-365) towards the appended dtype. */
int btm_int4_quantize(int device, void *stream, int N, int K, int group, const void *w_f16, void *out_packed,
                      void *out_scales_f16);

/* Element-wise dtype conversion among BTM_F32, BTM_F16 and BTM_BF16 with round-to-nearest-even, n contiguous
 * elements. Extends the reference's convert_gpu(), which handles Float32 <-> BFloat16 only and leaves other
 * pairs untouched (Tensor/TensorOps.cu:337-345); rounding as its __floats2bfloat162_rn (:72). */
int btm_convert(int device, void *stream, int src_dtype, int dst_dtype, int64_t n, const void *src, void *dst);

/* Unpack only: int8 out[n,k] = W[n,k] in [-8,7]. */
int btm_int4_unpack(int device, void *stream, int N, int K, const void *w_packed, void *out_i8);

/* N-sharded matmul with the all-gather fused into the epilogue: this rank holds all of A
 * and the column block B[:, rank*Nloc:(rank+1)*Nloc]; it computes C[:, that block] and
 * stores every finished tile into the full row-major C of EVERY rank through peer-mapped
 * pointers (`C_ranks[r]` is rank r's C base, valid on this device; ldc = nranks*Nloc or
 * more). Takes the place of the reference's only multi-GPU primitive, the whole-tensor
 * cudaMemcpyPeer of move_gpu_to_gpu (Tensor/TensorOps.cu:282-313). The caller provides
 * the cross-rank barrier before C is read. dtype BTM_F16 or BTM_BF16. */
int btm_gemm_nshard(int device, void *stream, int dtype, int M, int Nloc, int K, const void *A, int64_t lda,
                    const void *B_local, int64_t ldb, void *const *C_ranks, int64_t ldc, int rank, int nranks);

/* The same product with ONE outbound copy per tile instead of nranks - 1: every rank's C lives in memory bound to one
 * NVSwitch multicast object (btm_mc_* below), `C_multicast` is this rank's mapping of that object and `C_local` its
 * ordinary mapping of its own copy. The epilogue writes each finished tile with multimem stores to `C_multicast`; the
 * switch delivers it to all copies, this rank's included. Stores only: nothing is ever loaded through the multicast
 * mapping. BTM_ERR_UNSUPPORTED (nothing launched) unless K > 0, Nloc and ldc are multiples of 8 and the operands are
 * 16-byte aligned; callers fall back to btm_gemm_nshard. The caller provides the cross-rank barrier before C is read. */
int btm_gemm_nshard_mc(int device, void *stream, int dtype, int M, int Nloc, int K, const void *A, int64_t lda,
                       const void *B_local, int64_t ldb, void *C_local, void *C_multicast, int64_t ldc, int rank, int nranks);

/* Multicast memory for btm_gemm_nshard_mc, one process per GPU. No counterpart in the reference (its one multi-GPU
 * primitive is a whole-tensor peer copy, Tensor/TensorOps.cu:282-313).
 *   btm_mc_supported  1 if `device` can be a member of a multicast object, else 0.
 *   btm_mc_create     (one rank) creates the object for `nranks` devices and `bytes` per device and returns a POSIX
 *                     file descriptor for it; the caller passes that descriptor to the other processes (SCM_RIGHTS
 *                     over a Unix-domain socket) and closes its copy afterwards.
 *   btm_mc_import     (the other ranks) opens the object from the received descriptor.
 *   btm_mc_add_device (every rank) adds its device to the object. The caller then makes sure that EVERY rank has
 *                     done so successfully before any rank goes on, because a bind waits for the whole team.
 *   btm_mc_bind       (every rank) allocates `bytes` of its own memory, binds it at offset 0 and maps both.
 *                     Returns the two mappings.
 *   btm_mc_release    (every rank, behind a barrier, while all ranks are alive) unmaps, unbinds and frees. */
typedef struct btm_mc btm_mc;
int btm_mc_supported(int device);
int btm_mc_create(int device, int nranks, size_t bytes, btm_mc **out, int *export_fd);
int btm_mc_import(int device, int nranks, size_t bytes, int fd, btm_mc **out);
int btm_mc_add_device(btm_mc *h);
int btm_mc_bind(btm_mc *h, void **local_ptr, void **mc_ptr);
int btm_mc_release(btm_mc *h);

/* Placement helper for an operand that every rank needs whole (A of the N-sharded product) when each rank has
 * only a slice of it at hand: `bufs[r]` is rank r's copy of the operand (peer-mapped, as for btm_gemm_nshard), and the
 * byte range [offset_bytes, offset_bytes + bytes) of this rank's copy is sent to the same range of every other
 * rank's copy with one asynchronous copy per peer on `stream`. When all ranks have done this for their own ranges
 * and a cross-rank barrier has passed, every copy is complete: an all-gather by placement. Extends the reference's
 * move_gpu_to_gpu (Tensor/TensorOps.cu:282-313), which copies one whole tensor to one other GPU. */
int btm_replicate_rows(int device, void *stream, void *const *bufs, int rank, int nranks, size_t offset_bytes, size_t bytes);

/* CUDA IPC helpers so that one-process-per-GPU callers can build `C_ranks`:
 * btm_ipc_alloc allocates `bytes` of device memory and writes a 64-byte handle;
 * btm_ipc_open maps a peer's handle on `device`; btm_ipc_close / btm_ipc_free undo them.
 * (The reference is single-process and reaches peers with cudaDeviceEnablePeerAccess,
 * Tensor/TensorOps.cu:300-301.) */
int btm_ipc_alloc(int device, size_t bytes, void **ptr, unsigned char handle[64]);
int btm_ipc_open(int device, const unsigned char handle[64], void **ptr);
int btm_ipc_close(int device, void *ptr);
int btm_ipc_free(int device, void *ptr);

#ifdef __cplusplus
}
#endif
#endif /* BTM_H */
