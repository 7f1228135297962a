// Tensor-core GEMM for sm_100a: D[M,N] = A[M,K] (row-major) * B[K,N] (column- or row-major) (+ C),
// FP16 or BF16 inputs, FP32 accumulation in tensor memory, D (and C) FP32 or rounded once to FP16 / BF16.
//
// Stands in for the reference's GemmKernelTensorCore (nn_operators/gemm/tensor_core_gemm.h:101-399),
// a Turing mma.sync.m16n8k8 kernel with FP16 accumulation that is unfinished and disabled there.
// Nothing of that design carries over; this is a Blackwell pipeline:
//
//   warp 0      producer: one lane issues TMA tile loads (cp.async.bulk.tensor.2d, 128-byte swizzle,
//               this CTA only) of a 128 x 64 A tile and a BN x 64 B tile per stage into a ring of
//               shared-memory stages, signalling `full` mbarriers with the byte count;
//   warp 1      MMA: owns the tensor-memory allocation; one lane issues tcgen05.mma
//               (cta_group::1, kind::f16, M=128, N=BN, K=16; four per stage) reading the operands
//               straight from shared memory through matrix descriptors, accumulating in TMEM, and
//               tcgen05.commit to the stage's `empty` mbarrier / the accumulator's `ready` mbarrier;
//   warps 2-5   epilogue: tcgen05.ld the 128 x BN FP32 accumulator (each warp its 32-lane quadrant),
//               add C when given, store D with 128-bit writes.
//
// The CTA is persistent: tiles are dealt round-robin in an order that keeps concurrently running
// tiles on neighbouring A/B panels (L2 reuse), and the accumulator is double buffered in TMEM
// (2 x BN columns) so the epilogue of one tile overlaps the MMAs of the next.
//
// M, N and K tails: TMA zero-fills out-of-range rows/columns, zero K-columns add nothing, and the
// epilogue predicates its stores.  K must be a multiple of 8 (16-byte global row pitch for TMA), and so
// must N when B is row-major.
//
// B layouts.  Column-major B[K,N] (K contiguous, the layout the reference's kernel consumes after its
// ldmatrix.trans, tensor_core_gemm.h:171-179) is a K-major operand: one TMA box of BN rows x 64 K.
// Row-major B[K,N] (N contiguous) is an MN-major operand: BN/64 boxes of 64 K-rows x 64 columns, each
// 8 swizzle atoms (8 K-rows x 128 bytes) stacked along K; the matrix descriptor then steps 1024 bytes
// per 8 K and 8192 bytes per 64 columns, and the instruction descriptor marks B as MN-major.
//
// 16-bit output (the reference's ElementC = half, nn_operators/gemm/main.cu:190-192): the FP32
// accumulator (plus C, read in D's type) is rounded to nearest even once, in the epilogue.  The
// reference accumulates in FP16 inside mma.sync; that loss is not reproduced.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiting role records a code in the
// device status word, raises the CTA's abort flag and all roles drain and leave; tensor memory is
// released on every path.
#pragma once

#include <cuda.h>

#include "../../common/common.h"

namespace ko {
namespace tc {

constexpr int kBM = 128;          // rows of D per tile = TMEM lanes
constexpr int kBK = 64;           // K elements per stage: 64 * 2 B = one 128-byte swizzle row
constexpr int kUmmaK = 16;        // K per tcgen05.mma for 16-bit inputs
constexpr int kThreads = 192;     // 6 warps: producer, MMA, 4 x epilogue

// codes written to the status word (first failure wins)
enum : unsigned { kStatusOk = 0, kTimeoutProducer = 1, kTimeoutMma = 2, kTimeoutEpilogue = 3, kTimeoutDrain = 4 };

// MT: 128-row halves of the tile that share every B tile (1 or 2).  With MT = 2 a CTA computes 256 x BN: the
// operand bytes brought into shared memory per MMA drop by a third (A 32 KB + B 32 KB per 8 MMAs instead of
// A 16 KB + B 32 KB per 4), which is what limits the 128-row tile on long K; the two halves then fill tensor
// memory (2 x BN columns), so the epilogue of a tile no longer overlaps the next tile's MMAs.
// kBoxes: staging boxes per epilogue warp for the TMA stores of D (a store keeps its box until it has been read out
// of shared memory).  Two are in use; four, paid for with one stage of the operand ring, measured slower at every
// shape (FFN 16384 x 3072 x 768: 80.4 against 78.8 us), so the stores in flight are not what limits the epilogue.
template <int BN, int MT = 1, int kBoxes = 2>
struct TileConfig {
    static constexpr int kBN = BN;
    static constexpr int kBytesA = MT * kBM * kBK * 2;
    static constexpr int kBytesB = BN * kBK * 2;
    static constexpr int kStageBytes = kBytesA + kBytesB;
    static constexpr int kTmemCols = 2 * BN;  // MT = 1: double-buffered FP32 accumulator; MT = 2: one per half (power of two >= 32)
    static constexpr int kBarrierBytes = 256;
    // epilogue staging for TMA stores: per epilogue warp kBoxes 32-row x 32-column FP32 boxes (4 KB each)
    static constexpr int kStoreBoxes = kBoxes;
    static constexpr int kStoreBoxBytes = 32 * 32 * 4;
    static constexpr int kStoreBytes = 4 * kBoxes * kStoreBoxBytes;
    static constexpr int kSmemLimit = 232448;  // 227 KB: the most one CTA may use
    // + 1024 so the stage ring can be aligned to the 1024-byte swizzle period; as many stages as fit, at most 6
    static constexpr int kFit = (kSmemLimit - 1024 - kBarrierBytes - kStoreBytes) / kStageBytes;
    static constexpr int kStages = kFit > 6 ? 6 : kFit;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + kBarrierBytes + 1024;
    static_assert(BN == 64 || BN == 128 || BN == 256, "BN must keep 2*BN a power of two <= 512");
    static_assert(MT == 1 || MT == 2, "one or two 128-row halves");
    static_assert(kBoxes >= 2 && kBoxes <= 8, "staging boxes per epilogue warp");
    static_assert(kStages >= 2, "the operand ring needs at least two stages");
    static_assert(kSmemBytes <= kSmemLimit, "stage ring exceeds the shared memory of an SM");
};

// ------------------------------------------------------------------------------------------------
// thin PTX wrappers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// TMA 2-D tile load into this CTA's shared memory; x = innermost (K) coordinate, y = row
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// TMA 2-D tile store from this CTA's shared memory (bulk async-group completion)
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(src)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// until at most N of this thread's bulk groups are still READING their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// whole warp
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; accumulate == 0 overwrites D
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the mbarrier is arrived on once every tcgen05.mma issued so far by this thread has completed
// the same with the descriptors given as (low, high) words: the low word holds the start address (16-byte units, bits
// 0-13) and the leading offset, so stepping through a stage is one 32-bit add on it
__device__ __forceinline__ void umma_f16_words(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive FP32 columns: thread t receives row (lane base + t)
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// The same load without the wait: the registers may be read only after tmem_ld_wait().  Lets the load of the next
// 32 columns run while the current ones are written out.
__device__ __forceinline__ void tmem_ld_32x32_issue(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what the TMA load above produces): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);  // start address, 16-byte units
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzle): 1
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset: 8 rows * 128 B
    d |= (uint64_t)1 << 46;                        // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                        // layout: 128-byte swizzle
    return d;
}

// kind::f16 instruction descriptor: FP32 accumulator, A and B of `fmt` (0 = F16, 1 = BF16), both
// K-major, dense, M x N tile
__host__ __device__ constexpr uint32_t make_idesc(int fmt, int m, int n) {
    return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// tile order: groups of kGroupM tile-rows, tile-columns fastest inside a group's rows
constexpr int kGroupM = 8;
__device__ __forceinline__ void tile_coords(long long t, int tiles_m, int tiles_n, int &tm, int &tn) {
    // 32-bit division whenever the tile index allows: the 64-bit one is emulated, a few hundred nanoseconds on the
    // single thread that issues the MMAs, at every tile boundary
    const long long per_group = (long long)kGroupM * tiles_n;
    int group, in_group;
    if (t <= 0x7fffffffLL) {
        const unsigned tt = (unsigned)t, pg = (unsigned)per_group;
        group = (int)(tt / pg);
        in_group = (int)(tt - (unsigned)group * pg);
    } else {
        group = (int)(t / per_group);
        in_group = (int)(t % per_group);
    }
    const int first_m = group * kGroupM;
    const int rows_in_group = min(kGroupM, tiles_m - first_m);
    tm = first_m + in_group % rows_in_group;
    tn = in_group / rows_in_group;
}

struct GemmParams {
    int M, N, K;
    const void *C;    // may be null; same element type as D
    void *D;
    unsigned *status; // device status word
    int fmt;          // A and B: 0 = F16, 1 = BF16
    int out_fmt;      // D and C: 0 = FP32, 1 = F16, 2 = BF16
    int b_row_major;  // 0: B[K,N] column-major (K contiguous); 1: row-major (N contiguous)
    // Column tiles.  tiles_n == 0: every tile is BN columns wide (tiles_n = ceil(N / BN)).  Otherwise N is cut into
    // tiles_n tiles of which the first wide_tiles_n are bn_wide columns and the rest bn_narrow (both multiples of 32,
    // bn_narrow <= bn_wide <= BN; column-major B only): a tile count that fills the last wave of CTAs instead of
    // leaving part of it idle.  map_b then has a box of bn_wide rows and map_b_narrow one of bn_narrow rows.
    int tiles_n, wide_tiles_n, bn_wide, bn_narrow;
    // K slices (single-CTA kernel only).  split_k > 1: every tile is computed by split_k CTAs, each over a contiguous
    // range of K-blocks, and every CTA writes its FP32 partial tile to `partials` (one slot of kTileM x BN floats per
    // (tile, slice)) instead of D; gemm_slice_sum_kernel, launched behind this kernel, adds the slices in K order and
    // writes D.
    int split_k;
    float *partials;
};

// where column tile tn starts and how wide it is
template <int BN>
__device__ __forceinline__ void column_tile(const GemmParams &p, int tn, int &col0, int &bn) {
    if (p.tiles_n == 0) {
        col0 = tn * BN;
        bn = BN;
    } else if (tn < p.wide_tiles_n) {
        col0 = tn * p.bn_wide;
        bn = p.bn_wide;
    } else {
        col0 = p.wide_tiles_n * p.bn_wide + (tn - p.wide_tiles_n) * p.bn_narrow;
        bn = p.bn_narrow;
    }
}

// Tile t of a CTA's round-robin sequence -> (tile row, column tile).  With uneven column tiles all wide tiles come
// first (then the narrow ones), so that a CTA whose first tile is wide gets narrow ones afterwards; inside each of
// the two regions the order is tile_coords' (groups of kGroupM tile-rows, for L2 reuse).
__device__ __forceinline__ void tile_of(const GemmParams &p, long long t, int tiles_m, int tiles_n, int &tm, int &tn) {
    if (p.tiles_n == 0) {
        tile_coords(t, tiles_m, tiles_n, tm, tn);
        return;
    }
    const long long wide = (long long)tiles_m * p.wide_tiles_n;
    if (t < wide) {
        tile_coords(t, tiles_m, p.wide_tiles_n, tm, tn);
    } else {
        tile_coords(t - wide, tiles_m, tiles_n - p.wide_tiles_n, tm, tn);
        tn += p.wide_tiles_n;
    }
}


// MN-major operand tile made of 64-column blocks of 64 K-rows x 128 bytes (128-byte swizzle): 8-K-row
// atoms are 1024 bytes apart (stride offset), 64-column blocks 8192 bytes apart (leading offset).
__device__ __forceinline__ uint64_t smem_desc_mn_major_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)(8192 >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// two floats rounded to the 16-bit output type, low half first
__device__ __forceinline__ uint32_t pack16(float lo, float hi, int out_fmt) {
    if (out_fmt == 1) {
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
    const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&b);
}

// one thread's 32 consecutive columns of row `row`, starting at column `col`: D = acc (+ C), predicated on N
template <typename T>
__device__ __forceinline__ void store_row_segment(const float (&v)[32], const GemmParams &p, int row, int col) {
    constexpr int kVec = 16 / (int)sizeof(T);  // elements per 16-byte access
    const T *C = static_cast<const T *>(p.C);
    T *D = static_cast<T *>(p.D);
    const bool vec_ok = (p.N % kVec == 0) && ((reinterpret_cast<uintptr_t>(D) & 15u) == 0) &&
                        (C == nullptr || (reinterpret_cast<uintptr_t>(C) & 15u) == 0);
    const size_t off = (size_t)row * p.N + col;
    if (vec_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += kVec) {
            if (col + j < p.N) {
                alignas(16) T o[kVec];
                if (C) {
                    alignas(16) T c[kVec];
                    *reinterpret_cast<uint4 *>(c) = *reinterpret_cast<const uint4 *>(C + off + j);
#pragma unroll
                    for (int e = 0; e < kVec; ++e) o[e] = from_float<T>(v[j + e] + to_float(c[e]));
                } else {
#pragma unroll
                    for (int e = 0; e < kVec; ++e) o[e] = from_float<T>(v[j + e]);
                }
                *reinterpret_cast<uint4 *>(D + off + j) = *reinterpret_cast<const uint4 *>(o);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col + j < p.N) D[off + j] = from_float<T>(C ? v[j] + to_float(C[off + j]) : v[j]);
    }
}

// One 32 x 32 chunk of D from registers: lane = row row_base + lane, r = its 32 consecutive columns starting at column
// `col` (FP32 bits).  kTmaStore: registers -> swizzled shared box -> TMA store (box store_seq % kBoxes of this warp's
// kBoxes staging boxes of box_bytes each, store_seq counts the warp's stores across tiles); otherwise direct 16-byte
// stores (and + C).  Warp-collective.
template <bool kTmaStore, int kBoxes>
__device__ __forceinline__ void store_chunk(const CUtensorMap *map_d, const GemmParams &p, const uint32_t (&r)[32], int row_base,
                                            int col, int lane, uint32_t warp_boxes, uint32_t box_bytes, uint32_t &store_seq) {
    if constexpr (kTmaStore) {
        // row = lane, 8 chunks of 16 B, chunk j stored at j ^ (row & 7): conflict-free, and exactly the 128-byte
        // swizzle the store's tensor map undoes
        const uint32_t box = warp_boxes + (store_seq % kBoxes) * box_bytes;
        if (lane == 0) bulk_wait_group_read<kBoxes - 1>();  // the store issued from this box kBoxes chunks ago has read it
        __syncwarp();
        if (p.out_fmt == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t dst = box + (uint32_t)lane * 128u + (uint32_t)((j ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(r[4 * j]), "r"(r[4 * j + 1]),
                             "r"(r[4 * j + 2]), "r"(r[4 * j + 3])
                             : "memory");
            }
        } else {
            // 16-bit D: rows of 64 bytes, 4 chunks of 16 B, chunk j stored at j ^ ((row >> 1) & 3): the
            // 64-byte swizzle of the store's tensor map, conflict-free for 8 consecutive rows
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t dst = box + (uint32_t)lane * 64u + (uint32_t)((j ^ ((lane >> 1) & 3)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst),
                             "r"(pack16(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]), p.out_fmt)),
                             "r"(pack16(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]), p.out_fmt)),
                             "r"(pack16(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]), p.out_fmt)),
                             "r"(pack16(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]), p.out_fmt))
                             : "memory");
            }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            // rows / columns beyond M / N are clipped by the map; a box that lies entirely outside is
            // skipped, but still closes a (then empty) group so that the box rotation holds
            if (row_base < p.M && col < p.N) tma_store_2d(map_d, col, row_base, box);
            bulk_commit_group();
        }
        ++store_seq;
    } else {
        const int row = row_base + lane;
        if (row < p.M && col < p.N) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            if (p.out_fmt == 0) store_row_segment<float>(v, p, row, col);
            else if (p.out_fmt == 1) store_row_segment<__half>(v, p, row, col);
            else store_row_segment<__nv_bfloat16>(v, p, row, col);
        }
    }
}

// One epilogue warp's share of one 128-row block of a tile: its 32 accumulator rows (TMEM lanes of its quadrant),
// columns [0, bn) of the accumulator that starts at TMEM address t_row, written to D rows row_base .. row_base + 31,
// columns col0 .. col0 + bn - 1, chunk by chunk (store_chunk).  Warp-collective: all 32 lanes call it.
template <bool kTmaStore, int kBoxes>
__device__ __forceinline__ void epilogue_block(const CUtensorMap *map_d, const GemmParams &p, uint32_t t_row, int row_base,
                                               int col0, int bn, int lane, uint32_t warp_boxes, uint32_t box_bytes,
                                               uint32_t &store_seq) {
    if constexpr (kTmaStore) {
        // two register sets: the load of the next 32 columns is in flight while these are written out
        uint32_t ra[32], rb[32];
        tmem_ld_32x32_issue(t_row, ra);
#pragma unroll 1
        for (int c0 = 0; c0 < bn; c0 += 64) {
            tmem_ld_wait();
            if (c0 + 32 < bn) tmem_ld_32x32_issue(t_row + c0 + 32, rb);
            store_chunk<true, kBoxes>(map_d, p, ra, row_base, col0 + c0, lane, warp_boxes, box_bytes, store_seq);
            if (c0 + 32 < bn) {
                tmem_ld_wait();
                if (c0 + 64 < bn) tmem_ld_32x32_issue(t_row + c0 + 64, ra);
                store_chunk<true, kBoxes>(map_d, p, rb, row_base, col0 + c0 + 32, lane, warp_boxes, box_bytes, store_seq);
            }
        }
    } else {
#pragma unroll 1
        for (int c0 = 0; c0 < bn; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32_issue(t_row + c0, r);  // warp-collective: every lane takes part
            tmem_ld_wait();
            store_chunk<false, kBoxes>(map_d, p, r, row_base, col0 + c0, lane, warp_boxes, box_bytes, store_seq);
        }
    }
}

// One epilogue warp writes its 32 rows x bn columns of a K slice's accumulator into the slice's slot: 32 x 32 chunks
// of 4 KB, row-major inside a chunk (a lane's 32 columns are 128 contiguous bytes).
__device__ __forceinline__ void publish_block(float *slot_chunks, uint32_t t_row, int bn, int lane) {
#pragma unroll 1
    for (int c0 = 0; c0 < bn; c0 += 32) {
        float v[32];
        tmem_ld_32x32(t_row + c0, v);
        float4 *dst = reinterpret_cast<float4 *>(slot_chunks + ((size_t)(c0 >> 5) << 10) + lane * 32);
#pragma unroll
        for (int j = 0; j < 8; ++j) __stcg(dst + j, make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
    }
}

// kTmaStore: D is written by TMA stores staged through shared memory (needs a 16-byte row pitch and base for D
// and no C operand); otherwise every thread stores its row segment directly (and adds C when given)
template <int BN, bool kTmaStore, int MT = 1, int kBoxes = 2>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_b_narrow, const __grid_constant__ CUtensorMap map_d,
                    const GemmParams p) {
    using Cfg = TileConfig<BN, MT, kBoxes>;
    constexpr int kTileM = MT * kBM;
    extern __shared__ uint8_t ko_tc_smem_raw[];
    // stage ring on a 1024-byte boundary (swizzle period), barriers behind it
    const uint32_t raw = smem_u32(ko_tc_smem_raw);
    const uint32_t ring = (raw + 1023u) & ~1023u;
    uint8_t *ring_ptr = ko_tc_smem_raw + (ring - raw);
    const uint32_t store_base = ring + Cfg::kStages * Cfg::kStageBytes;  // 1024-byte aligned
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring_ptr + Cfg::kStages * Cfg::kStageBytes + Cfg::kStoreBytes);
    const uint32_t bar_base = store_base + Cfg::kStoreBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
    auto acc_ready_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::kStages + a); };
    auto acc_free_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::kStages + 2 + a); };
    const uint32_t drain_bar = bar_base + 8u * (2 * Cfg::kStages + 4);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * Cfg::kStages + 5);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.M + kTileM - 1) / kTileM, tiles_n = p.tiles_n ? p.tiles_n : (p.N + BN - 1) / BN;
    const int k_blocks = (p.K + kBK - 1) / kBK;
    // work units: (tile, K slice), the slices of a tile next to each other so that they run at the same time
    const int split = p.split_k > 1 ? p.split_k : 1;
    const long long num_units = (long long)tiles_m * tiles_n * split;
    auto unit_of = [&](long long u, long long &t, int &slice, int &kb0, int &kb1) {
        if (split == 1) {
            t = u; slice = 0; kb0 = 0; kb1 = k_blocks;
        } else {
            t = u / split;
            slice = (int)(u - t * split);
            kb0 = (int)((long long)k_blocks * slice / split);
            kb1 = (int)((long long)k_blocks * (slice + 1) / split);
        }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_ready_bar(a), 1);
            mbar_init(acc_free_bar(a), 4);  // one arrival per epilogue warp
        }
        mbar_init(drain_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        fence_proxy_async();
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        if (p.tiles_n) prefetch_tensormap(&map_b_narrow);
        if (kTmaStore) prefetch_tensormap(&map_d);
    }
    grid_launch_dependents();  // the stream's next kernel may set up while this one drains
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // launched with programmatic stream serialization: barriers, tensor memory and descriptor prefetch above
    // overlap the previous kernel's tail; operands and D are touched only after its writes are visible
    grid_dependency_wait();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0, stage = 0, fill = 0;  // K-blocks issued, ring position of the next one, times the ring went round
            bool ok = true;
            for (long long u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
                long long t;
                int slice, kb0, kb1, tm, tn, col0, bn;
                unit_of(u, t, slice, kb0, kb1);
                tile_of(p, t, tiles_m, tiles_n, tm, tn);
                column_tile<BN>(p, tn, col0, bn);
                const CUtensorMap *b_map = (p.tiles_n && bn != p.bn_wide) ? &map_b_narrow : &map_b;  // box of bn rows
                const uint32_t stage_bytes = (uint32_t)Cfg::kBytesA + (uint32_t)bn * (kBK * 2);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = (int)stage;
                    const uint32_t phase = fill & 1u;
                    if (++stage == (uint32_t)Cfg::kStages) { stage = 0; ++fill; }
                    if (!mbar_wait(empty_bar(s), phase ^ 1u, abort_flag)) {
                        if (!*abort_flag) atomicCAS(p.status, kStatusOk, kTimeoutProducer);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(full_bar(s), stage_bytes);
                    const uint32_t dst = ring + s * Cfg::kStageBytes;
                    tma_load_2d(dst, &map_a, kb * kBK, tm * kTileM, full_bar(s));  // one box of kTileM rows
                    if (!p.b_row_major) {
                        tma_load_2d(dst + Cfg::kBytesA, b_map, kb * kBK, col0, full_bar(s));
                    } else {
#pragma unroll
                        for (int nb = 0; nb < BN / 64; ++nb)
                            tma_load_2d(dst + Cfg::kBytesA + nb * 8192, &map_b, tn * BN + nb * 64, kb * kBK, full_bar(s));
                    }
                }
            }
            if (!ok) {
                // loads already issued still land in shared memory: wait (bounded) for the most recent
                // fill of every stage before the block may retire
                for (uint32_t back = 0; back < (uint32_t)Cfg::kStages && back < it; ++back) {
                    const uint32_t j = it - 1 - back;
                    const uint32_t bar = full_bar(j % Cfg::kStages), parity = (j / Cfg::kStages) & 1u;
                    for (uint32_t spin = 0; spin < kSpinLimit && !mbar_try_wait(bar, parity); ++spin) {}
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0, local_tile = 0;
            uint32_t stage = 0, phase = 0;  // ring position of K-block `it` and the parity of its fill
            // Shared-memory descriptors as two words (smem_desc_k_major_sw128 / smem_desc_mn_major_sw128 of the ring's
            // first stage): the high word (stride 1024 bytes, version, 128-byte swizzle) is the same for every operand,
            // the low word is the address in 16-byte units plus the leading offset (1 for K-major, 8192 bytes for a
            // row-major B).  Building them per MMA cost the issuing thread about 75 cycles per instruction.
            const uint32_t desc_hi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
            const uint32_t a_lo0 = ((ring & 0x3ffffu) >> 4) | (1u << 16);
            const uint32_t b_lo0 = (((ring + Cfg::kBytesA) & 0x3ffffu) >> 4) | (p.b_row_major ? (uint32_t)(8192 >> 4) << 16 : 1u << 16);
            const uint32_t b_kstep = p.b_row_major ? 2048u >> 4 : (uint32_t)(kUmmaK * 2) >> 4;
            bool ok = true;
            for (long long u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++local_tile) {
                long long t;
                int slice, kb0, kb1, tm, tn, col0, bn;
                unit_of(u, t, slice, kb0, kb1);
                tile_of(p, t, tiles_m, tiles_n, tm, tn);
                column_tile<BN>(p, tn, col0, bn);
                const uint32_t idesc = make_idesc(p.fmt, kBM, bn) | (p.b_row_major ? 1u << 16 : 0u);  // bit 16: B is MN-major
                // MT = 1: two accumulators used in turn; MT = 2: one accumulator per half, both busy with every tile
                const uint32_t acc = MT == 1 ? (local_tile & 1u) : 0u, acc_phase = (MT == 1 ? (local_tile >> 1) : local_tile) & 1u;
                if (!mbar_wait(acc_free_bar(acc), acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    // descriptors of this stage: the ring's plus the stage's offset in 16-byte units
                    const uint32_t a_lo = a_lo0 + stage * (uint32_t)(Cfg::kStageBytes >> 4), b_lo = b_lo0 + stage * (uint32_t)(Cfg::kStageBytes >> 4);
                    uint32_t accumulate = kb != kb0 ? 1u : 0u;
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k) {
                        // advancing K inside the swizzled row: +32 bytes per 16 elements (K-major); row-major B: 16 K-rows
                        // further = two 8-row atoms = 2048 bytes
                        umma_f16_words(d_tmem, a_lo + k * 2, desc_hi, b_lo + k * b_kstep, desc_hi, idesc, accumulate);
                        if (MT == 2)  // rows 128..255 of the tile: 16 KB further in the stage, accumulator columns BN..2BN-1
                            umma_f16_words(d_tmem + BN, a_lo + (kBM * kBK * 2 >> 4) + k * 2, desc_hi, b_lo + k * b_kstep, desc_hi, idesc, accumulate);
                        accumulate = 1u;
                    }
                    umma_commit(empty_bar(stage));  // the stage is reusable once these MMAs have read it
                    if (++stage == (uint32_t)Cfg::kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) umma_commit(acc_ready_bar(acc));
            }
            if (!ok) {
                if (!*abort_flag) atomicCAS(p.status, kStatusOk, kTimeoutMma);
                *abort_flag = 1;
            }
            // nothing may still be writing tensor memory when it is released
            umma_commit(drain_bar);
            bool drained = false;
            for (uint32_t spin = 0; spin < kSpinLimit && !(drained = mbar_try_wait(drain_bar, 0)); ++spin) {}
            if (!drained) atomicCAS(p.status, kStatusOk, kTimeoutDrain);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may read
        uint32_t local_tile = 0;
        uint32_t store_seq = 0;  // TMA stores issued by this warp so far: store n uses staging box n % kBoxes
        bool ok = true;
        for (long long u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++local_tile) {
            long long t;
            int slice, kb0, kb1, tm, tn, col0, bn;
            unit_of(u, t, slice, kb0, kb1);
            tile_of(p, t, tiles_m, tiles_n, tm, tn);
            column_tile<BN>(p, tn, col0, bn);
            const uint32_t acc = MT == 1 ? (local_tile & 1u) : 0u, acc_phase = (MT == 1 ? (local_tile >> 1) : local_tile) & 1u;
            if (!mbar_wait(acc_ready_bar(acc), acc_phase, abort_flag)) {
                if (lane == 0 && !*abort_flag) atomicCAS(p.status, kStatusOk, kTimeoutEpilogue);
                *abort_flag = 1;
                ok = false;
                break;
            }
            tc_fence_after();
            if (split > 1) {
                // a K slice: the partial tile goes to its slot, gemm_slice_sum_kernel writes D
                constexpr size_t kSlotFloats = (size_t)kTileM * BN;
                float *slot = p.partials + ((size_t)t * split + slice) * kSlotFloats;
#pragma unroll 1
                for (int half = 0; half < MT; ++half) {
                    const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (MT == 1 ? acc * BN : half * BN);
                    publish_block(slot + ((size_t)((half * 4 + quad) * (BN / 32)) << 10), t_row, bn, lane);
                }
            } else {
#pragma unroll 1
                for (int half = 0; half < MT; ++half) {
                    const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + (MT == 1 ? acc * BN : half * BN);
                    epilogue_block<kTmaStore, kBoxes>(&map_d, p, t_row, tm * kTileM + half * kBM + quad * 32, col0, bn, lane,
                                                      store_base + (uint32_t)((warp - 2) * kBoxes) * Cfg::kStoreBoxBytes,
                                                      (uint32_t)Cfg::kStoreBoxBytes, store_seq);
                }  // halves
            }
            // the accumulator buffer may be overwritten once all four warps have read it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_free_bar(acc));
        }
        // shared memory must outlive the reads of the stores still in flight
        if (kTmaStore && lane == 0) bulk_wait_group_read<0>();
        __syncwarp();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// Second step of a GEMM cut into K slices: D = sum over the slices of a tile, in K order, (+ C), rounded once to D's
// type.  One block per 32 x 32 chunk of a tile (the unit gemm_tcgen05_kernel's epilogue warps write): thread i takes
// columns 4 * (i % 8) .. + 3 of row i / 8, so a warp reads 512 contiguous bytes of every slice and writes four
// 128-byte row segments of D.  tile_m / bn_full: the first kernel's tile (kTileM x BN).
// (a template only so that the header may be included by several translation units)
template <int kBlock = 256>
__global__ void __launch_bounds__(kBlock) gemm_slice_sum_kernel(const GemmParams p, int tile_m, int bn_full) {
    static_assert(kBlock == 256, "one thread per float4 of a 32 x 32 chunk");
    const int chunks_n = bn_full / 32, chunks_per_tile = (tile_m / 32) * chunks_n;
    const long long t = blockIdx.x / chunks_per_tile;
    const int chunk = (int)(blockIdx.x - t * chunks_per_tile);
    const int tiles_m = (p.M + tile_m - 1) / tile_m, tiles_n = p.tiles_n ? p.tiles_n : (p.N + bn_full - 1) / bn_full;
    int tm, tn, col0, bn;
    tile_of(p, t, tiles_m, tiles_n, tm, tn);
    if (p.tiles_n == 0) {
        col0 = tn * bn_full;
        bn = bn_full;
    } else {
        column_tile<0>(p, tn, col0, bn);
    }
    const int row = tm * tile_m + (chunk / chunks_n) * 32 + (int)threadIdx.x / 8;
    const int c_in_tile = (chunk % chunks_n) * 32 + ((int)threadIdx.x & 7) * 4;
    const int col = col0 + c_in_tile;
    grid_launch_dependents();
    grid_dependency_wait();  // the slices are complete and visible
    if (c_in_tile >= bn || row >= p.M || col >= p.N) return;
    const size_t slot_floats = (size_t)tile_m * bn_full;
    const float4 *src = reinterpret_cast<const float4 *>(p.partials + (size_t)t * p.split_k * slot_floats + ((size_t)chunk << 10)) + threadIdx.x;
    // four slices' loads in flight at a time (they are independent), added in slice order
    const size_t slot_vecs = slot_floats / 4;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < p.split_k; s0 += 4) {
        float4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (s0 + i < p.split_k) v[i] = __ldcg(src + (size_t)(s0 + i) * slot_vecs);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (s0 + i < p.split_k) {
                if (s0 + i == 0) sum = v[0];
                else { sum.x += v[i].x; sum.y += v[i].y; sum.z += v[i].z; sum.w += v[i].w; }
            }
    }
    float v[4] = {sum.x, sum.y, sum.z, sum.w};
    const size_t off = (size_t)row * p.N + col;
    const bool whole = col + 4 <= p.N;
    if (p.out_fmt == 0) {
        const float *C = static_cast<const float *>(p.C);
        float *D = static_cast<float *>(p.D);
        if (whole && p.N % 4 == 0 && (reinterpret_cast<uintptr_t>(D) & 15u) == 0 && (C == nullptr || (reinterpret_cast<uintptr_t>(C) & 15u) == 0)) {
            if (C) {
                const float4 c = *reinterpret_cast<const float4 *>(C + off);
                v[0] += c.x; v[1] += c.y; v[2] += c.z; v[3] += c.w;
            }
            *reinterpret_cast<float4 *>(D + off) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
            for (int e = 0; e < 4 && col + e < p.N; ++e) D[off + e] = C ? v[e] + C[off + e] : v[e];
        }
    } else if (p.out_fmt == 1) {
        const __half *C = static_cast<const __half *>(p.C);
        __half *D = static_cast<__half *>(p.D);
        for (int e = 0; e < 4 && col + e < p.N; ++e) D[off + e] = __float2half_rn(C ? v[e] + __half2float(C[off + e]) : v[e]);
    } else {
        const __nv_bfloat16 *C = static_cast<const __nv_bfloat16 *>(p.C);
        __nv_bfloat16 *D = static_cast<__nv_bfloat16 *>(p.D);
        for (int e = 0; e < 4 && col + e < p.N; ++e) D[off + e] = __float2bfloat16_rn(C ? v[e] + __bfloat162float(C[off + e]) : v[e]);
    }
}

}  // namespace tc
}  // namespace ko
