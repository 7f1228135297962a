// Source-level GemmKernelTensorCore (the reference's template, nn_operators/gemm/tensor_core_gemm.h:101-399): same
// template parameters, static members and call operator, so
//   gemm<GemmKernelTensorCore<half, half, half, GemmShape<128,128,32>, GemmShape<64,64,32>, GemmShape<16,8,8>, 8, 8, 8>>
//       <<<grid, K::thread_per_block, K::smem_total_size_in_bytes, stream>>>(problem, A, B, C, D)
// compiles and produces D = A * B (+ C) for row-major A [M,K], B [K,N], C / D [M,N], as the reference intends (its own
// kernel is an unfinished Turing mma.sync design with FP16 accumulation and a wrong epilogue, disabled at
// nn_operators/gemm/main.cu:344).  As the reference's driver does for every kernel, the launcher raises the kernel's
// dynamic shared-memory limit when smem_total_size_in_bytes exceeds 48 KB (nn_operators/gemm/main.cu:75-82).
//
// With 16-bit A and B, a 128-row thread-block shape of 64 / 128 / 256 columns and four warps the product runs on the
// 5th-generation tensor cores WITHOUT any host-built descriptor: all threads copy the operand tiles with cp.async
// straight into the 128-byte-swizzled shared-memory layouts the MMA reads (A as a K-major tile, row-major B as an
// MN-major tile of 64-column blocks), one thread issues tcgen05.mma (M = 128, N = BN, K = 16) with matrix descriptors
// built in the kernel, the FP32 accumulator lives in tensor memory and the four warps read it back with tcgen05.ld.
// Three stages; a stage is refilled once the MMAs that read it have completed (tcgen05.commit on an mbarrier).
// Needs K % 8 == 0, N % 8 == 0 and 16-byte aligned A and B (16-byte copies); anything else, and every other
// instantiation, multiplies on the FP32 pipe through a shared tile.  Accumulation is FP32 either way (the reference
// accumulates in FP16).  Waits are bounded; one that runs out abandons the call's remaining tiles.
//
// The library's own tensor-core path (TMA-fed, persistent, two-SM capable) is behind the C ABI: ko_gemm_tc and friends.
#pragma once

#include "../../common/common.h"
#include "tensor_core_gemm.h"

// ---------------------------------------------------------------------------------------------
// Warp-level primitives under the reference's names (nn_operators/gemm/tensor_core_gemm.h:30-99): MMA<16,8,8> is one
// mma.sync m16n8k8 with FP16 operands AND FP16 accumulation, LDMatrix<N, transpose> one ldmatrix of N 8x8 tiles of
// 16-bit elements.  Same call operators (untyped pointers to the lane's fragment registers / to the lane's row in shared
// memory).  They are the legacy tensor path, kept for code written against the reference's header; nothing in this
// library's own GEMMs uses them (those run on tcgen05).  Fragment layouts are PTX's: for m16n8k8, lane l holds A rows
// l/4 and l/4+8, columns 2(l%4)..+1; B row (k) 2(l%4)..+1, column l/4; C and D rows l/4 and l/4+8, columns 2(l%4)..+1.
// ---------------------------------------------------------------------------------------------
template <int M, int N, int K>
struct MMA;

template <>
struct MMA<16, 8, 8> {
    __device__ __forceinline__ void operator()(void *ptr_A, void *ptr_B, void *ptr_C, void *ptr_D) const {
        const uint32_t *a = static_cast<const uint32_t *>(ptr_A);
        const uint32_t b = *static_cast<const uint32_t *>(ptr_B);
        const uint32_t c0 = static_cast<const uint32_t *>(ptr_C)[0], c1 = static_cast<const uint32_t *>(ptr_C)[1];  // C may alias D
        uint32_t d0, d1;
        asm volatile("mma.sync.aligned.m16n8k8.row.col.f16.f16.f16.f16 {%0, %1}, {%2, %3}, {%4}, {%5, %6};"
                     : "=r"(d0), "=r"(d1)
                     : "r"(a[0]), "r"(a[1]), "r"(b), "r"(c0), "r"(c1));
        static_cast<uint32_t *>(ptr_D)[0] = d0;
        static_cast<uint32_t *>(ptr_D)[1] = d1;
    }
};

template <int N, bool transpose>
struct LDMatrix {
    static_assert(N == 1 || N == 2 || N == 4, "ldmatrix loads one, two or four 8x8 tiles");
    // data_ptr: N 32-bit registers of this lane; smem_ptr: the 16-byte row this lane addresses (lanes 0..8N-1 count)
    __device__ __forceinline__ void operator()(void *data_ptr, void *smem_ptr) const {
        uint32_t *d = static_cast<uint32_t *>(data_ptr);
        const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(smem_ptr));
        if constexpr (N == 1) {
            if constexpr (transpose) asm volatile("ldmatrix.sync.aligned.x1.trans.m8n8.shared.b16 {%0}, [%1];" : "=r"(d[0]) : "r"(addr));
            else asm volatile("ldmatrix.sync.aligned.x1.m8n8.shared.b16 {%0}, [%1];" : "=r"(d[0]) : "r"(addr));
        } else if constexpr (N == 2) {
            if constexpr (transpose)
                asm volatile("ldmatrix.sync.aligned.x2.trans.m8n8.shared.b16 {%0, %1}, [%2];" : "=r"(d[0]), "=r"(d[1]) : "r"(addr));
            else asm volatile("ldmatrix.sync.aligned.x2.m8n8.shared.b16 {%0, %1}, [%2];" : "=r"(d[0]), "=r"(d[1]) : "r"(addr));
        } else {
            if constexpr (transpose)
                asm volatile("ldmatrix.sync.aligned.x4.trans.m8n8.shared.b16 {%0, %1, %2, %3}, [%4];"
                             : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                             : "r"(addr));
            else
                asm volatile("ldmatrix.sync.aligned.x4.m8n8.shared.b16 {%0, %1, %2, %3}, [%4];"
                             : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                             : "r"(addr));
        }
    }
};

template <typename ElementA_, typename ElementB_, typename ElementC_, typename ThreadBlockShape_, typename WarpShape_,
          typename InstructionShape_, int AlignmentA, int AlignmentB, int AlignmentC>
struct GemmKernelTensorCore {
    using ElementA = ElementA_;
    using ElementB = ElementB_;
    using ElementC = ElementC_;
    using ThreadBlockShape = ThreadBlockShape_;
    using WarpShape = WarpShape_;
    using InstructionShape = InstructionShape_;

    static constexpr int kTileK = 16;  // FP32-pipe path: K per shared tile
    static constexpr int warp_count_m = ThreadBlockShape::kM / WarpShape::kM;
    static constexpr int warp_count_n = ThreadBlockShape::kN / WarpShape::kN;
    static constexpr int warp_count = warp_count_m * warp_count_n;
    static constexpr int thread_per_block = warp_count * 32;
    // tensor-core path: 16-bit operands of one type, 128 x {64,128,256} tile, four warps (one per TMEM lane quadrant)
    static constexpr bool kTensorPath =
        std::is_same<ElementA, ElementB>::value && (std::is_same<ElementA, half>::value || std::is_same<ElementA, __nv_bfloat16>::value) &&
        ThreadBlockShape::kM == 128 && (ThreadBlockShape::kN == 64 || ThreadBlockShape::kN == 128 || ThreadBlockShape::kN == 256) &&
        thread_per_block == 128;
    static constexpr int kStages = 3, kBlockK = 64;  // tensor-core path: 64 K per stage = one 128-byte swizzle row
    static constexpr int kStageBytesA = ThreadBlockShape::kM * kBlockK * 2, kStageBytesB = kBlockK * ThreadBlockShape::kN * 2;
    static constexpr int kSimtBytesA = ThreadBlockShape::kM * kTileK * (int)sizeof(float);
    static constexpr int kSimtBytesB = kTileK * ThreadBlockShape::kN * (int)sizeof(float);
    static constexpr int smem_A_total_size_in_bytes = kTensorPath ? kStages * kStageBytesA : kSimtBytesA;
    static constexpr int smem_B_total_size_in_bytes = kTensorPath ? kStages * kStageBytesB : kSimtBytesB;
    // tensor-core path: + 1024 to align the ring to the swizzle period, + 64 for mbarriers and the TMEM address
    static constexpr int smem_total_size_in_bytes = smem_A_total_size_in_bytes + smem_B_total_size_in_bytes + (kTensorPath ? 1024 + 64 : 0);

    __device__ static float widen(const float &v) { return v; }
    __device__ static float widen(const half &v) { return __half2float(v); }
    __device__ static float widen(const __nv_bfloat16 &v) { return __bfloat162float(v); }
    template <typename T>
    __device__ static T narrow(float v) {
        if constexpr (sizeof(T) == 4) return v;
        else if constexpr (std::is_same<T, half>::value) return __float2half_rn(v);
        else return __float2bfloat16_rn(v);
    }

    // 16 bytes global -> shared, zero-filled when !valid
    __device__ static void copy16(uint32_t dst, const void *src, bool valid) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0) : "memory");
    }

    // tcgen05 path (see the header comment); called by all 128 threads of every block
    __device__ __forceinline__ void run_tensor_cores(const shape::GemmCoord &problem_size, ElementA *ptr_A, ElementB *ptr_B,
                                                     ElementC *ptr_C, ElementC *ptr_D) const {
        namespace tc = ko::tc;
        constexpr int BM = ThreadBlockShape::kM, BN = ThreadBlockShape::kN;
        constexpr int kStageBytes = kStageBytesA + kStageBytesB;
        constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;
        extern __shared__ uint8_t ko_tc_src_smem[];
        const uint32_t raw = ko::smem_u32(ko_tc_src_smem);
        const uint32_t ring = (raw + 1023u) & ~1023u;
        uint8_t *ring_ptr = ko_tc_src_smem + (ring - raw);
        const uint32_t bar_base = ring + kStages * kStageBytes;
        auto done_bar = [&](int s) { return bar_base + 8u * s; };  // the MMAs that read stage s have completed
        const uint32_t acc_bar = bar_base + 8u * kStages;          // all MMAs of the tile have completed
        uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(ring_ptr + kStages * kStageBytes + 8 * (kStages + 1));

        const int M = (int)problem_size.m(), N = (int)problem_size.n(), K = (int)problem_size.k();
        const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
        const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
        const int k_blocks = (K + kBlockK - 1) / kBlockK;
        const int fmt = std::is_same<ElementA, half>::value ? 0 : 1;
        const uint32_t idesc = tc::make_idesc(fmt, BM, BN) | (1u << 16);  // B is MN-major (row-major [K, N])

        if (tid == 0) {
            for (int s = 0; s <= kStages; ++s) ko::mbar_init(bar_base + 8u * s, 1);
            ko::fence_barrier_init();
        }
        if (warp == 0) tc::tmem_alloc(ko::smem_u32(tmem_slot), kTmemCols);
        tc::tc_fence_before();
        __syncthreads();
        tc::tc_fence_after();
        const uint32_t tmem_base = *tmem_slot;

        // Stage fill: A tile [BM rows][64 K] as a K-major tile -- row r, 16-byte chunk c at (r/8)*1024 + (r%8)*128 +
        // ((c ^ r%8) << 4); B tile [64 K][BN] as an MN-major tile -- 64-column block nb, K-row k, chunk c of its 128 bytes
        // at nb*8192 + (k/8)*1024 + (k%8)*128 + ((c ^ k%8) << 4).  Out-of-range rows, columns and K read as zero.
        auto fill = [&](int stage, int m0, int n0, int k0) {
            const uint32_t a_dst = ring + stage * kStageBytes, b_dst = a_dst + kStageBytesA;
#pragma unroll
            for (int i = 0; i < BM * 8 / 128; ++i) {
                const int e = tid + i * 128, r = e >> 3, c = e & 7;
                const int gm = m0 + r, gk = k0 + c * 8;
                const bool ok = gm < M && gk < K;
                copy16(a_dst + (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)),
                       ptr_A + (ok ? (size_t)gm * K + gk : 0), ok);
            }
#pragma unroll
            for (int i = 0; i < kBlockK * (BN / 8) / 128; ++i) {
                const int e = tid + i * 128, k = e / (BN / 8), cc = e % (BN / 8);  // cc: 16-byte chunk along N
                const int nb = cc >> 3, c = cc & 7;
                const int gk = k0 + k, gn = n0 + cc * 8;
                const bool ok = gk < K && gn < N;
                copy16(b_dst + (uint32_t)(nb * 8192 + (k >> 3) * 1024 + (k & 7) * 128 + ((c ^ (k & 7)) << 4)),
                       ptr_B + (ok ? (size_t)gk * N + gn : 0), ok);
            }
        };
        auto bounded_wait = [&](uint32_t bar, uint32_t parity) -> bool {
            bool ok = false;
            for (uint32_t spin = 0; spin < ko::kSpinLimit && !(ok = ko::mbar_try_wait(bar, parity)); ++spin) {}
            return ok;
        };

        uint32_t it = 0;        // K-blocks consumed so far by this block (over all its tiles): stage = it % kStages
        uint32_t tile_count = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < tiles_m * tiles_n && alive; tile += gridDim.x, ++tile_count) {
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            // prologue: kStages - 1 K-blocks in flight (a stage is refilled only after the MMAs that read it)
            for (int p = 0; p < kStages - 1; ++p) {
                if (p < k_blocks) {
                    const uint32_t use = it + p;
                    if (use >= (uint32_t)kStages) alive = alive && bounded_wait(done_bar(use % kStages), ((use / kStages) - 1) & 1u);
                    fill(use % kStages, m0, n0, p * kBlockK);
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 2) : "memory");  // this thread's copies of K-block kb landed
                ko::fence_proxy_async();  // make them visible to the tensor core's (async proxy) reads
                __syncthreads();          // ... everybody's
                const int s = it % kStages;
                if (tid == 0) {
                    tc::tc_fence_after();
                    const uint32_t a_addr = ring + s * kStageBytes, b_addr = a_addr + kStageBytesA;
#pragma unroll
                    for (int k = 0; k < kBlockK / tc::kUmmaK; ++k)
                        tc::umma_f16(tmem_base, tc::smem_desc_k_major_sw128(a_addr + k * tc::kUmmaK * 2),
                                     tc::smem_desc_mn_major_sw128(b_addr + k * 2048), idesc, (kb | k) != 0 ? 1u : 0u);
                    tc::umma_commit(done_bar(s));
                    if (kb == k_blocks - 1) tc::umma_commit(acc_bar);
                }
                // refill the stage that K-block kb - 1 used with K-block kb + kStages - 1
                const int next = kb + kStages - 1;
                if (next < k_blocks) {
                    const uint32_t use = it + kStages - 1;
                    if (use >= (uint32_t)kStages) alive = alive && bounded_wait(done_bar(use % kStages), ((use / kStages) - 1) & 1u);
                    fill(use % kStages, m0, n0, next * kBlockK);
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            // epilogue: thread (warp, lane) owns row m0 + 32 * warp + lane
            alive = alive && bounded_wait(acc_bar, tile_count & 1u);
            alive = __syncthreads_and(alive) != 0;
            if (alive) {
                tc::tc_fence_after();
                tc::GemmParams prm{};
                prm.M = M; prm.N = N; prm.K = K; prm.C = ptr_C; prm.D = ptr_D;
                const int row = m0 + warp * 32 + lane;
                const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    float v[32];
                    tc::tmem_ld_32x32(t_row + c0, v);
                    if (row < M && n0 + c0 < N) tc::store_row_segment<ElementC>(v, prm, row, n0 + c0);
                }
            }
            tc::tc_fence_before();
            __syncthreads();  // the accumulator is free for the next tile's MMAs
        }
        // every MMA this block issued has completed (its last tile's acc_bar was waited for, or the block gave up and
        // no further MMA was issued): tensor memory can go back
        if (warp == 0) {
            tc::tc_fence_after();
            tc::tmem_dealloc(tmem_base, kTmemCols);
        }
    }

    __device__ __forceinline__ void operator()(const shape::GemmCoord &problem_size, ElementA *ptr_A, ElementB *ptr_B,
                                               ElementC *ptr_C, ElementC *ptr_D) const {
        constexpr int BM = ThreadBlockShape::kM, BN = ThreadBlockShape::kN;
        if constexpr (kTensorPath) {
            const bool copies_ok = problem_size.k() % 8 == 0 && problem_size.n() % 8 == 0 &&
                                   (reinterpret_cast<uintptr_t>(ptr_A) & 15u) == 0 && (reinterpret_cast<uintptr_t>(ptr_B) & 15u) == 0;
            if (copies_ok && blockDim.x == 128) {  // uniform over the grid
                run_tensor_cores(problem_size, ptr_A, ptr_B, ptr_C, ptr_D);
                return;
            }
        }
        extern __shared__ __align__(16) float ko_tc_compat_smem[];
        float *As = ko_tc_compat_smem;           // [BM][kTileK]
        float *Bs = ko_tc_compat_smem + BM * kTileK;  // [kTileK][BN]
        const int M = (int)problem_size.m(), N = (int)problem_size.n(), K = (int)problem_size.k();
        const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
        constexpr int kOutputs = BM * BN;
        constexpr int kPerThread = (kOutputs + thread_per_block - 1) / thread_per_block;
        for (int tile = blockIdx.x; tile < tiles_m * tiles_n; tile += gridDim.x) {
            const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
            float acc[kPerThread];
#pragma unroll
            for (int i = 0; i < kPerThread; ++i) acc[i] = 0.f;
            for (int k0 = 0; k0 < K; k0 += kTileK) {
                __syncthreads();
                for (int e = threadIdx.x; e < BM * kTileK; e += blockDim.x) {
                    const int m = e / kTileK, k = e % kTileK;
                    As[e] = (m0 + m < M && k0 + k < K) ? widen(ptr_A[(size_t)(m0 + m) * K + k0 + k]) : 0.f;
                }
                for (int e = threadIdx.x; e < kTileK * BN; e += blockDim.x) {
                    const int k = e / BN, n = e % BN;
                    Bs[e] = (k0 + k < K && n0 + n < N) ? widen(ptr_B[(size_t)(k0 + k) * N + n0 + n]) : 0.f;
                }
                __syncthreads();
#pragma unroll
                for (int i = 0; i < kPerThread; ++i) {
                    const int o = threadIdx.x + i * blockDim.x;
                    if (o < kOutputs) {
                        const int m = o / BN, n = o % BN;
#pragma unroll
                        for (int k = 0; k < kTileK; ++k) acc[i] = fmaf(As[m * kTileK + k], Bs[k * BN + n], acc[i]);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < kPerThread; ++i) {
                const int o = threadIdx.x + i * blockDim.x;
                const int m = m0 + o / BN, n = n0 + o % BN;
                if (o < kOutputs && m < M && n < N) {
                    float v = acc[i];
                    if (ptr_C) v += widen(ptr_C[(size_t)m * N + n]);
                    ptr_D[(size_t)m * N + n] = narrow<ElementC>(v);
                }
            }
        }
    }
};
