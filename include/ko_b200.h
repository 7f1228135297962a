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
 *   - operator entry points take DEVICE pointers valid on the CURRENT device, enqueue on
 *     `stream` (a cudaStream_t passed as void*, NULL = default stream) and return without
 *     synchronising; they allocate nothing;
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
 * last poll, KO_OK otherwise.  No counterpart in the reference, whose kernels never wait. */
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
 * y = (x - mean) * rsqrt(var + eps) [* gamma] [+ beta]; statistics in FP32 by Welford/Chan
 * merging; var = M2 / (cols - ddof), ddof in {0, 1}.  gamma and beta may each be NULL and have
 * the I/O element type.  `out` may equal `in`.
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
 * the operator runs and `out` is copied back, cut into `chunks` row ranges (0 = 8, at most 64) that
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
 * The first call on a (device, stream) that needs partial-tile scratch allocates it with cudaMalloc.
 * ---------------------------------------------------------------------------------------- */
int ko_sgemm_f32(int64_t M, int64_t N, int64_t K, const float *A, const float *B, const float *C,
                 float *D, void *stream);

/* Same operation and kernel as ko_sgemm_f32 for hosts that must not allocate device memory (a process
 * whose own pool owns the whole GPU, a loop that cannot afford an allocation's implicit
 * synchronisation, code running where the allocation calls are forbidden).  It has no counterpart
 * in the reference.  The split-K partial tiles and arrival counters live in a fixed array inside the
 * library image -- 2 Mi floats (8 MiB) and 4096 counters per GPU, held until the process exits --
 * and no cudaMalloc / cudaFree or allocating library routine is called.
 *   split_k  0 = choose (never more slices than the fixed scratch holds), 1 = no split (needs no
 *            scratch, any size), n > 1 = exactly n K-slices; a request that needs more than the
 *            scratch holds (tiles * split_k * 16384 floats, tiles = ceil(M/128) * ceil(N/128), at most
 *            4096 tiles) returns KO_ERR_SHAPE and launches nothing.
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

#ifdef __cplusplus
}
#endif
#endif /* KO_B200_H */
