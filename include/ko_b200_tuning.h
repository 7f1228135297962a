/*
 * ko_b200_tuning.h -- launch-geometry overrides of the operator entry points of ko_b200.h (same
 * semantics; a zero knob selects the library's default).  For sweeps and for tests that pin every
 * instantiated kernel variant; applications call the plain entry points.  The reference fixes these
 * choices as template arguments and <<<grid, block>>> literals in its drivers
 * (nn_operators/softmax/main.cu:77, nn_operators/layernorm/main.cu:75-76, nn_operators/gemm/main.cu:343).
 */
#ifndef KO_B200_TUNING_H
#define KO_B200_TUNING_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* knobs of the row operators; pass NULL for all defaults */
typedef struct ko_row_knobs {
    int tier;            /* 0 = choose, 1 = warp, 2 = block, 3 = stream (scalar), 4 = staged (TMA ring),
                            5 = resident (LayerNorm only: persistent blocks, packed FP32 math),
                            6 = cluster (one row per thread-block cluster, partials through DSMEM; softmax: stages = 1
                                turns the shared-memory prefetch of the next row's slice off),
                            7 = prefetching block (softmax only: row in registers, next row bulk-copied to shared memory),
                            8 = reread (FP32 softmax and every LayerNorm: one row per block in two passes, the second served
                                by the L2; block = 256 / 512 / 1024 threads, grid_cap = rows in flight),
                            9 = lane groups (LayerNorm rows of at most 128 vectors: a row per group of stage_rows = 4 / 8 /
                                16 / 32 lanes with up to four vectors each, rows_per_warp row slots per group, persistent
                                warps with gamma and beta held in registers) */
    int rows_per_warp;   /* warp / staged tier: independent row slots a warp processes together (a slot is
                            one row per group of 8, 16 or 32 lanes, i.e. 4, 2 or 1 rows); LayerNorm reread tier:
                            1 = one row per block at a time, 2 = two (gamma / beta loaded once for both),
                            0 = two from 512 KB per row */
    int block;           /* warp tier: threads per block (<= 256); block / resident tier: threads per row (128..1024, a power
                            of two; the resident tier also takes 768 and 896: four vectors per thread through the shared-memory ring) */
    int64_t grid_cap;    /* warp / block / stream tier: upper bound on the grid (0 = one pass per warp) */
    int stage_rows;      /* staged tier: rows per bulk copy (0 = about 16-32 KB) */
    int stages;          /* staged tier: ring depth (0 = fill about 100 KB); LayerNorm resident tier: 1 = the block's next
                            row prefetched into registers, 3 = its next rows in flight into shared memory (cp.async), 0 = choose;
                            reread tier: 1 = direct loads, 3 = loads through a shared-memory ring of items, 0 = choose */
    int ctas_per_sm;     /* staged tier: persistent blocks per SM (0 = 1) */
    int cluster;         /* cluster tier: blocks per cluster, 2 / 4 / 8 (0 = smallest that holds the row) */
} ko_row_knobs_t;

int ko_softmax_f32_tuned(const float *in, float *out, int64_t rows, int32_t cols, const ko_row_knobs_t *knobs,
                         void *stream);
int ko_layernorm_f32_tuned(const float *in, float *out, int64_t rows, int32_t cols, float eps, const float *gamma,
                           const float *beta, int ddof, const ko_row_knobs_t *knobs, void *stream);
int ko_layernorm_f16_tuned(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, float eps,
                           const uint16_t *gamma, const uint16_t *beta, int ddof, const ko_row_knobs_t *knobs,
                           void *stream);
int ko_layernorm_bf16_tuned(const uint16_t *in, uint16_t *out, int64_t rows, int32_t cols, float eps,
                            const uint16_t *gamma, const uint16_t *beta, int ddof, const ko_row_knobs_t *knobs,
                            void *stream);
/* variant: 0 = choose, 1..3 = scalar-FFMA tilings (128x128, 128x64, 64x64), 4 = packed-FFMA 128x128 kernel;
 * 6 / 7 / 8 = variant 4 pinned to 128x128 tiles with 128-thread
 * blocks / 128x128 tiles with two warp groups that halve the block's K range / 64x128 tiles with four
 * warp groups that quarter it; split_k (variants 4, 6, 7, 8): 0 = choose the block count (stream-K),
 * 1 = one block per tile, n > 1 = n K-slices per tile */
int ko_sgemm_f32_tuned(int64_t M, int64_t N, int64_t K, const float *A, const float *B, const float *C, float *D,
                       int variant, int split_k, void *stream);
/* fmt: 0 = F16, 1 = BF16 (A, B); out_fmt: 0 = FP32, 1 = F16, 2 = BF16 (D, C); b_row_major: 0 / 1; bn: 0 = choose,
 * 64 / 128 / 256 = columns of D per 128-row tile, 512 = the 256 x 256 tile (two 128-row halves per CTA share each B tile),
 * all with equal column tiles; 1024 / 1280 = the 128- / 256-row tile with N cut into uneven column tiles of at most 256
 * columns that fill the last round of CTAs (KO_ERR_SHAPE when the tiles fit one round anyway; 0 uses them when the cost
 * model predicts a gain);
 * 2048 = the two-SM kernel (tcgen05 cta_group::2: a pair of CTAs per 256 x 256 tile, either B layout), 2304 = the same
 * with uneven column tiles (column-major B only);
 * bits 16-23 of bn, added to one of the codes above (single-CTA kernels, i.e. not 2048 / 2304): K slices per tile,
 * 0 = choose (slices only when bn is 0 too), 1 = none, n <= 64 = n slices (at most K / 64 rounded up) whose FP32 partial
 * tiles go through the context's scratch lane of `stream` and are added in K order by a second kernel;
 * store_mode: 0 = choose, 1 = TMA-store epilogue (KO_ERR_SHAPE when not possible), 2 = direct stores */
int ko_gemm_tc_tuned(int fmt, int out_fmt, int b_row_major, int64_t M, int64_t N, int64_t K, const void *A, const void *B,
                     const void *C, void *D, int bn, int store_mode, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* KO_B200_TUNING_H */
