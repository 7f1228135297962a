/*
 * ko_b200.h -- C ABI of the B200 (sm_100a) operator library: row softmax, Welford LayerNorm
 * forward, FP32 FFMA SGEMM and the FP16/BF16-in FP32-accumulate tcgen05 GEMM, plus the
 * host/device Tensor buffer, seeded fills and host-side comparison metrics.
 *
 * The reference project (donglinz/kernel_optimization) has no FFI: its operator API is C++
 * templates with compile-time shapes launched with <<<>>> from three drivers.  Each entry point
 * below names the reference interface it stands in for (file:line inside that project).
 *
 * Conventions
 *   - every function returns a ko_status_t (0 = success); nothing prints, exits or aborts;
 *     ko_last_error_string() gives the calling thread's most recent failure in words;
 *   - operator entry points take DEVICE pointers valid on the CURRENT device and enqueue on
 *     `stream` (a cudaStream_t passed as void*, NULL = default stream);
 *   - a WARMED operator call enqueues and returns: it does not synchronise, allocate or change
 *     host-side state, and may therefore be captured into a CUDA graph.  The first call of a kind
 *     does set-up that must not happen inside a capture, so make it eagerly beforehand:
 *       every operator   the first launch of a kernel needing more than 48 KB of shared memory
 *                        raises that kernel's limit (once per kernel and device);
 *       ko_sgemm_f32     the first call on a (context, stream) that splits K allocates that stream's
 *                        scratch lane with cudaMalloc (see ko_context_create below); later calls on
 *                        that stream reuse it;
 *       ko_gemm_*        a combination of (pointer, shape, type) not seen before encodes its TMA
 *                        descriptors (host work only, no device call); a problem of few tiles and long K
 *                        is cut into K slices and uses the same per-stream scratch lane as
 *                        ko_sgemm_f32 -- inside a capture on a stream whose lane does not exist yet
 *                        it runs unsliced instead;
 *       ko_*_f32_host    the first call on a device creates two copy streams and their events;
 *                        these calls also take one process-wide lock while they enqueue;
 *       ko_sgemm_f32_no_alloc  looks up its scratch address on first use per device (see there);
 *   - matrices are dense (leading dimension = logical width);
 *   - there is no CPU fallback: without a usable CUDA device the operator calls fail.
 */
#ifndef KO_B200_H
#define KO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ko_status {
    KO_OK = 0,
    KO_ERR_INVALID_ARG = 1, /* NULL pointer, negative size, unknown flag */
    KO_ERR_ALIGN = 2,       /* pointer or row pitch not aligned as the kernel requires */
    KO_ERR_SHAPE = 3,       /* shape outside what the kernel supports */
    KO_ERR_CUDA = 4,        /* a CUDA runtime/driver call failed (see ko_last_error_string) */
    KO_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up (status word set by the kernel) */
    KO_ERR_NO_DEVICE = 6    /* no sm_100 device is current */
} ko_status_t;

const char *ko_status_string(int status);
const char *ko_last_error_string(void);
/* major*10000 + minor*100 + patch */
int ko_version(void);
/* Kernels built on mbarrier / tcgen05 pipelines bound every device-side wait; one that runs out
 * records a code in a device status word instead of hanging.  This call waits for the device's
 * outstanding work, returns KO_ERR_TIMEOUT (and clears the words) if any kernel gave up since the
 * last poll, KO_OK otherwise.  "Waits" is a cudaDeviceSynchronize(): every stream of the current
 * device, blocking or not, has drained when the words are read, so a code written by any kernel
 * enqueued before the call is seen by it.  No counterpart in the reference, whose kernels never wait. */
int ko_poll_device_status(void);
/* Exercises that path without any fault: launches a one-warp kernel that waits at most `polls`
 * (1 .. 2^20) polls on an mbarrier nothing arrives at, lets the wait run out and records a code;
 * the next ko_poll_device_status() returns KO_ERR_TIMEOUT.  No counterpart in the reference. */
int ko_selftest_bounded_wait(unsigned polls, void *stream);

/* ------------------------------------------------------------------------------------------
 * Tensor: paired host (pinned) + device byte buffer.
 * Stands in for class Tensor, common/tensor.h:11-40 and common/tensor.cu:8-42.
 * ---------------------------------------------------------------------------------------- */
typedef struct ko_tensor ko_tensor_t;

/* Tensor::Tensor(size_t) tensor.cu:8-11; device < 0 means the current device */
int ko_tensor_create(size_t size_in_bytes, int device, ko_tensor_t **out);
/* Tensor::~Tensor tensor.cu:23-26 */
int ko_tensor_destroy(ko_tensor_t *t);
/* Tensor::host_ref<T>() tensor.h:20-23 */
void *ko_tensor_host_ptr(ko_tensor_t *t);
/* Tensor::device_ref<T>() tensor.h:25-28 */
void *ko_tensor_device_ptr(ko_tensor_t *t);
size_t ko_tensor_size_in_bytes(const ko_tensor_t *t);
int ko_tensor_device(const ko_tensor_t *t);
/* Tensor::host_to_device / host_to_device_async tensor.cu:28-34 */
int ko_tensor_host_to_device(ko_tensor_t *t);
int ko_tensor_host_to_device_async(ko_tensor_t *t, void *stream);
/* Tensor::device_to_host / device_to_host_async tensor.cu:36-42 */
int ko_tensor_device_to_host(ko_tensor_t *t);
int ko_tensor_device_to_host_async(ko_tensor_t *t, void *stream);

/* ------------------------------------------------------------------------------------------
 * Seeded host fills.  Stand in for the inline fill loops of the reference drivers
 * (nn_operators/softmax/main.cu:31-36, nn_operators/gemm/main.cu:46-66), which draw from a
 * default-seeded std::default_random_engine and are not reproducible by specification.
 * Element i depends only on (seed, tensor_id, elem_offset + i): Philox4x32-10 keyed by
 * (seed, tensor_id), counter = element index / 4.  Values are generated in float64 and rounded
 * once to the storage type.  dtype: 0 = f32, 1 = f16, 2 = bf16 (16-bit types as raw uint16).
 * ---------------------------------------------------------------------------------------- */
enum { KO_DTYPE_F32 = 0, KO_DTYPE_F16 = 1, KO_DTYPE_BF16 = 2 };

int ko_fill_uniform(void *host_dst, int dtype, int64_t n, uint32_t seed, uint32_t tensor_id,
                    int64_t elem_offset, float lo, float hi);
int ko_fill_normal(void *host_dst, int dtype, int64_t n, uint32_t seed, uint32_t tensor_id,
                   int64_t elem_offset, float mean, float stddev);
/* rows are numbered row_offset + r; within every `block` consecutive rows, every column
 * c > (row % block) is overwritten with `value` (FP32 only) */
int ko_fill_causal_mask_f32(float *host_dst, int64_t rows, int32_t cols, int64_t row_offset,
                            int32_t block, float value);

/* ------------------------------------------------------------------------------------------
 * Host-side comparison ("check") of a result against expected values supplied by the caller.
 * Stands in for the element loop of nn_operators/gemm/main.cu:157-176 (|got - ref| > 1e-3).
 * These compare buffers; they never compute the operator on the CPU.
 * ---------------------------------------------------------------------------------------- */
int ko_check_max_abs_f32(const float *got, const float *want, int64_t n, double *out);
/* max |got - want| / max(|want|, floor) */
int ko_check_max_rel_f32(const float *got, const float *want, int64_t n, double floor, double *out);
/* ||got - want||_F / ||want||_F */
int ko_check_rel_frobenius_f32(const float *got, const float *want, int64_t n, double *out);
/* max over rows of |sum(row) - 1| */
int ko_check_max_rowsum_err_f32(const float *got, int64_t rows, int32_t cols, double *out);

/* ------------------------------------------------------------------------------------------
 * Row softmax over the last dimension, FP32, row-major [rows, cols].
 * Stands in for softmax<SoftMaxWarpImpl|SoftMaxBlockImpl|SoftMaxBlockNoCacheImpl<float, vec,
 * rows, cols>><<<grid, block, smem, stream>>>(in, out): nn_operators/softmax/softmax.h:11-60,
 * :62-113, :116-166, :168-174 (launched at nn_operators/softmax/main.cu:58-60).
 * Computes exp(x - rowmax) / sum.  `out` may equal `in`.  Any cols >= 1; the 128-bit path needs
 * cols % 4 == 0 and 16-byte aligned pointers, other inputs take a scalar path.
 * ---------------------------------------------------------------------------------------- */
int ko_softmax_f32(const float *in, float *out, int64_t rows, int32_t cols, void *stream);
/* FP16 / BF16 in and out (raw uint16 storage), FP32 arithmetic, one rounding on store: the element
 * type the reference's Exp<half> (common/functors.h:71-77) and numeric_limits<half>
 * (common/common.h:171-177) provide for and its driver never instantiates.  The 128-bit path needs
 * cols % 8 == 0 and 16-byte aligned pointers. */
int ko_softmax_f16(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, void *stream);
int ko_softmax_bf16(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, void *stream);

/* ------------------------------------------------------------------------------------------
 * LayerNorm forward over the last dimension, row-major [rows, cols].
 * Stands in for layer_normalization<LayerNormWarpImpl|LayerNormBlockImpl|
 * LayerNormBlockNoCacheImpl<E, vec, rows, cols, affine>><<<...>>>(in, out, eps, gamma, beta):
 * nn_operators/layernorm/layernorm.h:145-201, :204-252, :254-300, :302-312.
 * y = (x - mean) * rsqrt(var + eps) [* gamma] [+ beta]; var = M2 / (cols - ddof), ddof in {0, 1};
 * statistics in FP32.  Which form of them runs depends on the row length only: rows a lane group
 * or a warp holds unpacked in registers (FP32 up to 1024 columns, 16-bit up to 1024) and the rows
 * of the resident tier (to 16384 columns) use the exact two-pass form over registers -- the mean from the
 * row sum, then M2 as the sum of squared deviations from that mean, i.e. the value the merge of
 * Welford triples converges to; longer rows (block, cluster, two-pass and scalar tiers) form
 * per-thread (count, mean, M2) triples and merge them pairwise (Chan et al.) across lanes, warps
 * and blocks.  Rows too long for one block's registers are read twice, the second time from the L2.
 * gamma and beta may each be NULL and have the I/O element type.  `out` may equal `in`.
 * ---------------------------------------------------------------------------------------- */
int ko_layernorm_f32(const float *in, float *out, int64_t rows, int32_t cols, float eps,
                     const float *gamma, const float *beta, int ddof, void *stream);
/* BF16 in/out (raw uint16 storage), FP32 statistics */
int ko_layernorm_bf16(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, float eps,
                      const uint16_t *gamma, const uint16_t *beta, int ddof, void *stream);
/* FP16 in/out (the reference's Rsqrt<half>, common/functors.h:105-111), FP32 statistics */
int ko_layernorm_f16(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, float eps,
                     const uint16_t *gamma, const uint16_t *beta, int ddof, void *stream);

/* ------------------------------------------------------------------------------------------
 * The same operators for a caller whose rows live in HOST memory: `in` is copied to the device,
 * the operator runs and `out` is copied back, cut into `chunks` nominal row ranges (0 = 8, at most 60;
 * from 4 on, the first and last range are each cut further into a quarter, a quarter and a half, so that
 * the stretches in which only one direction of the link is busy are short) that
 * flow through three streams, so that the copy in, the kernel and the copy out of neighbouring
 * chunks overlap and a call costs about one direction of the PCIe link.  Ordered like any other
 * work on `stream` (it starts after what `stream` holds and `stream` continues after the last
 * copy).  The tensors' first rows*cols elements are used; both must live on the current device;
 * gamma and beta are DEVICE pointers.  No counterpart in the reference, whose drivers copy whole
 * tensors before and after the launch (nn_operators/softmax/main.cu:38, :55, :62).
 * ---------------------------------------------------------------------------------------- */
int ko_softmax_f32_host(ko_tensor_t *in, ko_tensor_t *out, int64_t rows, int32_t cols, int chunks,
                        void *stream);
int ko_layernorm_f32_host(ko_tensor_t *in, ko_tensor_t *out, int64_t rows, int32_t cols, float eps,
                          const float *gamma, const float *beta, int ddof, int chunks, void *stream);

/* ------------------------------------------------------------------------------------------
 * SGEMM: D[M,N] = A[M,K] * B[K,N] (+ C[M,N] when C != NULL), all row-major FP32, FP32 FFMA.
 * Stands in for gemm<GemmKernelSimt<float,float,float,GemmShape<64,64,8>,GemmShape<32,32,8>,
 * 4,4,4>><<<grid, 128, smem, stream>>>(GemmCoord, A, B, C, D): nn_operators/gemm/gemm.h:11-21,
 * nn_operators/gemm/simt_gemm.h:46-375 (launched at nn_operators/gemm/main.cu:111-117).
 * Any M, N, K >= 1 (edges are predicated).  D must not alias A or B; D may equal C.
 * Every output is a chain of FP32 FMAs in ascending k, as in the reference; depending on the shape the
 * K range of a tile may be cut into parts that are accumulated that way and then added in K order
 * (deterministic: the same call gives the same bits; relative Frobenius error <= 1e-6 either way).
 * Partial tiles of a split K live in a scratch lane owned by a context (below), one lane per stream:
 * the first call on a stream that splits K allocates the lane with cudaMalloc, at the largest size
 * the shape rules can ask for (4 x SMs partial tiles of 64 KB, about 39 MB on a B200), and nothing
 * is freed or moved until the context is destroyed -- a graph captured after that first call keeps
 * valid pointers.  A captured launch and an eager launch on the SAME stream use the same lane:
 * replaying such a graph on another stream while that stream is busy races on it.
 * ---------------------------------------------------------------------------------------- */
int ko_sgemm_f32(int64_t M, int64_t N, int64_t K, const float *A, const float *B, const float *C,
                 float *D, void *stream);

/* ------------------------------------------------------------------------------------------
 * Context: the owner of what the launchers keep between calls -- the SGEMM's split-K scratch lanes
 * and the cache of encoded TMA descriptors of the tensor-core GEMM.  The plain entry points use a
 * default context per device (created on first use, kept until the process exits); a caller that
 * wants to bound or release that memory creates its own and calls the *_ctx forms.  No counterpart
 * in the reference, whose kernels need neither scratch nor descriptors.
 * ---------------------------------------------------------------------------------------- */
typedef struct ko_context ko_context_t;
/* device < 0 = the current device.  Creating a context allocates nothing on the device. */
int ko_context_create(int device, ko_context_t **out);
/* Waits for the context's device to drain (cudaDeviceSynchronize), then frees every scratch block
 * and forgets the cached descriptors.  Graphs captured from calls on this context must not be
 * replayed afterwards.  NULL is a no-op. */
int ko_context_destroy(ko_context_t *ctx);
/* Bytes of device memory the context holds, cached descriptors, cache hits and misses; ctx = NULL
 * reports the current device's default context; any out pointer may be NULL. */
int ko_context_stats(ko_context_t *ctx, size_t *device_bytes, size_t *tensor_maps, size_t *map_hits,
                     size_t *map_misses);
/* ko_sgemm_f32 / ko_gemm_tc on an explicit context (ctx = NULL: the default one).  The context's
 * device must be the current device. */
int ko_sgemm_f32_ctx(ko_context_t *ctx, int64_t M, int64_t N, int64_t K, const float *A,
                     const float *B, const float *C, float *D, void *stream);
int ko_gemm_tc_ctx(ko_context_t *ctx, int in_fmt, int out_fmt, int b_row_major, int64_t M, int64_t N,
                   int64_t K, const void *A, const void *B, const void *C, void *D, void *stream);

/* Same operation and kernel as ko_sgemm_f32 for hosts that must not allocate device memory (a process
 * whose own pool owns the whole GPU, a loop that cannot afford an allocation's implicit
 * synchronisation, code running where the allocation calls are forbidden).  It has no counterpart
 * in the reference.  The split-K partial tiles and arrival counters live in a fixed array inside the
 * library image -- 2 Mi floats (8 MiB: 128 partial tiles of 128 x 128) and 128 counters per GPU, held
 * until the process exits -- and no cudaMalloc / cudaFree or allocating library routine is called.
 *   split_k  0 = choose (never more slices than the fixed scratch holds), 1 = no split (needs no
 *            scratch, any size), n > 1 = exactly n K-slices.  A split needs tiles * split_k partial
 *            tiles, tiles = ceil(M/128) * ceil(N/128): at most 128 in all (64 tiles in 2 slices, 32 in
 *            4, ...); a request beyond that returns KO_ERR_SHAPE and launches nothing.
 * The first call on each device looks up the array's device address and configures the kernel; make
 * that call during set-up, before any stream capture.  Every call on a device uses the same array,
 * which keeps the previous call's contents (counters are cleared on `stream` before each launch):
 * calls whose kernels may overlap on the GPU race and must be ordered by the caller. */
int ko_sgemm_f32_no_alloc(int64_t M, int64_t N, int64_t K, const float *A, const float *B,
                          const float *C, float *D, int split_k, void *stream);

/* ------------------------------------------------------------------------------------------
 * Tensor-core GEMM: D[M,N] (row-major) = A[M,K] (row-major) * B[K,N] (+ C[M,N] when C != NULL);
 * FP16 or BF16 inputs as raw uint16, FP32 accumulate in tensor memory (tcgen05.mma), TMA-fed.
 * Stands in for gemm<GemmKernelTensorCore<half,half,half,GemmShape<128,128,32>,
 * GemmShape<64,64,32>,GemmShape<16,8,8>,8,8,8>>: nn_operators/gemm/tensor_core_gemm.h:101-399
 * (disabled call at nn_operators/gemm/main.cu:344).
 *
 * B is column-major in the named entry points, i.e. element (k,n) at B[n*K + k] (what the
 * reference's kernel multiplies after its transposing ldmatrix, tensor_core_gemm.h:171-179);
 * ko_gemm_tc also takes the reference driver's row-major B[K,N] (element (k,n) at B[k*N + n],
 * nn_operators/gemm/main.cu:201-203) with b_row_major = 1.
 * D and C are FP32 (.._f32) or the input type (.._f16 / .._bf16: the reference's ElementC = half,
 * nn_operators/gemm/main.cu:190-192; the FP32 sum plus C is rounded to nearest even once).
 * Requires K % 8 == 0 (and N % 8 == 0 for row-major B) and 16-byte aligned A and B; M, N, K tails
 * are handled; an unaligned or odd-pitch D falls back from 16-byte to scalar stores.
 * A problem whose tiles fill less than the device and whose K is long is computed as K slices: the
 * tensor-core kernel writes FP32 partial tiles to the context's scratch and a second kernel adds
 * them in K order (deterministic) and rounds once; the result then differs from the unsliced one
 * by FP32 summation order only.
 * ---------------------------------------------------------------------------------------- */
int ko_gemm_f16_f32(int64_t M, int64_t N, int64_t K, const uint16_t *A, const uint16_t *B,
                    const float *C, float *D, void *stream);
int ko_gemm_bf16_f32(int64_t M, int64_t N, int64_t K, const uint16_t *A, const uint16_t *B,
                     const float *C, float *D, void *stream);
int ko_gemm_f16_f16(int64_t M, int64_t N, int64_t K, const uint16_t *A, const uint16_t *B,
                    const uint16_t *C, uint16_t *D, void *stream);
int ko_gemm_bf16_bf16(int64_t M, int64_t N, int64_t K, const uint16_t *A, const uint16_t *B,
                      const uint16_t *C, uint16_t *D, void *stream);
/* in_fmt: 0 = FP16, 1 = BF16 (A and B); out_fmt: 0 = FP32, 1 = FP16, 2 = BF16 (D and C);
 * b_row_major: 0 = column-major B, 1 = row-major B. */
int ko_gemm_tc(int in_fmt, int out_fmt, int b_row_major, int64_t M, int64_t N, int64_t K,
               const void *A, const void *B, const void *C, void *D, void *stream);

/* ------------------------------------------------------------------------------------------
 * Probes of the source-level helper templates (kernel_optimization_b200/common/{common,functors}.h
 * and the Welford combiners of nn_operators/layernorm/layernorm.h).  The reference exposes these
 * helpers only as device templates; each probe instantiates them in a small kernel and runs them
 * on DEVICE buffers of the caller, so that a host can check them against its own arithmetic.
 * ---------------------------------------------------------------------------------------- */
/* Functors of common/functors.h:13-301 applied elementwise: out[i] = F(a[i] [, b[i] [, c[i]]]).
 * functor: 0 ReduceMax, 1 ReduceSum, 2 Exp, 3 Rsqrt, 4 Add, 5 Subtract, 6 Multiply, 7 Divide,
 *          8 MultiplyAdd (a * b + c);
 * form:    0 scalar functor F<T>; 1 F<AlignedArray<T, 16 / sizeof(T)>> on (vector, vector);
 *          2 the same on (vector, scalar), binary functors only: vector i is paired with b[i];
 * dtype:   KO_DTYPE_F32 / F16 / BF16 (16-bit types compute in their own precision, as the
 *          reference's half specialisations do).  Vector forms need n % (16 / sizeof(T)) == 0. */
int ko_probe_functor(int functor, int form, int dtype, const void *a, const void *b, const void *c,
                     void *out, int64_t n, void *stream);
/* kind 0: WarpReduce<Op, float> (common/common.h:37-46): groups x 32 inputs, out[g] read from lane 0;
 * kind 1: BlockReduce<Op, float> (:48-65) with `width` threads per block (32..1024, multiple of 32),
 *         run twice on the same cache: out[g] = first result, out[groups + g] = second, thread 0;
 * kind 2: to_scalar<Op<float>, float, 4> (:138-149): groups x 4 inputs;
 * kind 3: WarpReduce<ReduceMax, int32_t> from the identity -numeric_limits<int32_t>::max()
 *         (:151-178) over the inputs rounded to integers.
 * op: 0 = ReduceMax, 1 = ReduceSum. */
int ko_probe_reduce(int kind, int op, const float *in, float *out, int64_t groups, int width,
                    void *stream);
/* limits::numeric_limits<float | int32_t | half | __nv_bfloat16>::max() as device code sees them
 * (common/common.h:151-178); 16-bit values as raw bits. */
int ko_probe_limits(float *f32_max, int32_t *i32_max, uint16_t *f16_max, uint16_t *bf16_max,
                    void *stream);
/* Welford helpers over the rows of in[rows, cols]; out[rows, 3] = (count, mean, M2), M2 = sum of
 * squared deviations.  kind 0: WelfordUpdate<float> serially (nn_operators/layernorm/layernorm.h:13-23);
 * 1: 32-element chunks joined by WelfordMerge (:36-50); 2: WelfordUpdate<AlignedArray<float,4>>
 * (:25-34) + WelfordWarpAllReduce (:80-91), read from lane 31; 3: + WelfordWarpReduce, six-argument
 * form (:64-78), lane 0; 4: scalar updates + in-place WelfordWarpReduce (:52-62), lane 0;
 * 5: WelfordBlockAllReduce (:128-143) with `block` threads, read from the last thread;
 * 6: WelfordBlockReduce (:93-126), thread 0.  Kinds 2, 3, 5, 6 need cols % 4 == 0. */
int ko_probe_welford(int kind, const float *in, int64_t rows, int32_t cols, float *out, int block,
                     void *stream);
/* A whole row operator written only with those helper names, one block of `block` threads per row:
 * op 0 = softmax (ReduceMax / Subtract / Exp / ReduceSum / Divide, to_scalar, BlockReduce),
 * op 1 = LayerNorm with population variance (WelfordUpdate, WelfordBlockAllReduce, Rsqrt, Subtract,
 * Multiply, MultiplyAdd; gamma and beta both NULL or both given).  cols % 4 == 0. */
int ko_probe_composed_rowop(int op, const float *in, float *out, int64_t rows, int32_t cols,
                            float eps, const float *gamma, const float *beta, int block, void *stream);

/* gemm<GemmKernelTensorCore<half, half, half, GemmShape<128,128,32>, GemmShape<64,64,32>, GemmShape<16,8,8>, 8,8,8>>
 * launched as the reference's driver would launch it (nn_operators/gemm/main.cu:179-339, call disabled at :344):
 * half A [M,K], B [K,N], optional C and D [M,N], all row-major; D = A * B (+ C) with FP32 accumulation. */
int ko_probe_gemm_tensor_core_template(int64_t M, int64_t N, int64_t K, const uint16_t *A, const uint16_t *B,
                                       const uint16_t *C, uint16_t *D, void *stream);

/* One warp computes D[16,8] = A[16,K] * B[K,8] + C with the reference's warp-level helpers in the call shapes of its
 * warp loop (nn_operators/gemm/tensor_core_gemm.h:207, :218, :231): LDMatrix<2,false> for A, LDMatrix<1,true> for B,
 * MMA<16,8,8> with FP16 accumulation.  FP16 storage, everything row-major, K a multiple of 8 in [8, 64]. */
int ko_probe_mma_ldmatrix(const uint16_t *A, const uint16_t *B, const uint16_t *C, uint16_t *D, int32_t K, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* KO_B200_H */
