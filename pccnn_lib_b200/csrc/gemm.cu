// Dense contraction on the 5th-generation tensor cores:  C[M, N] (fp32) = A[M, K] * B[N, K]^T.
//
// This is the contraction of the convolutions (out = P * W, pccnn_lib_ops/pcconvs/kpconv.cu:55-59
// and mcconv.cu:63-70 of phermosilla/pccnn_lib, and dP = g * W^T of kpconv.cu:95-96), which the
// reference hands to cuBLAS SGEMM.
//
// Operands are bf16, K-contiguous ("K-major"), with rows padded to a multiple of 64 elements.
// fp32 accuracy comes from a split: x = hi + lo with hi = bf16(x), lo = bf16(x - hi), and three
// tensor-core passes hi*hi + lo*hi + hi*lo accumulated in the same fp32 accumulator; the
// dropped lo*lo term is below 2^-16 relative.  One pass serves bf16 inputs.
//
// Kernel: one CTA per 128 x BN output tile, 128 threads.
//   warp 0, one lane : TMA producer  -- cp.async.bulk.tensor 2-D loads of 128 x 64 (A) and BN x 64 (B)
//                      bf16 boxes, 128-byte swizzle, into a 2-4 stage ring, completion on mbarriers;
//                      with the split a stage carries the hi and lo planes of both operands
//   warp 1, one lane : MMA issuer    -- tcgen05.mma.cta_group::1.kind::f16, four K=16 steps per stage
//                      (x3 products with the split, all from the same shared-memory tiles),
//                      accumulator [128 lanes x BN columns] fp32 in tensor memory; tcgen05.commit
//                      releases the stage and finally signals the epilogue
//   all four warps   : epilogue      -- tcgen05.ld 32 lanes x 32 columns per warp and step, plain
//                      global stores of whole 128-byte row segments
// With more output tiles than SMs the persistent form runs instead (gemm_bf16_persistent_kernel below:
// one CTA per SM, accumulator double-buffered in tensor memory, four dedicated epilogue warps).
// Every wait is bounded: on expiry the kernel records a status word,
// leaves its loops, releases tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>

#include "common.cuh"
#include "gemm.cuh"
#include "tc_ptx.cuh"

namespace pccnn {

// Poll limit of every wait (about 2^21 polls are tens of milliseconds) and a test hook: a producer that stops
// issuing loads from a given K block on, so that a test can watch the consumers' waits run out with no copy in
// flight.  Both are read once per kernel; pccnn_gemm_set_test_hooks changes them.
__device__ uint32_t d_poll_limit = 1u << 21;
__device__ int d_withhold_from = -1;

// One accumulator segment of 32 columns (starting at column col0) of output row `row`: fp32 or bf16 stores,
// 128-bit wide where the destination allows.
__device__ __forceinline__ void store_acc_segment(const uint32_t (&r)[32], int row, int M, int N, int col0, float* C,
                                                  int ldc, int c_is_bf16) {
    if (row < M && c_is_bf16) {
        // bf16 output (inference configuration): C is a __nv_bfloat16 matrix, ldc in elements
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(C) + (size_t)row * ldc + col0;
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            const int col = col0 + j;
            if (col + 7 < N && ((((uintptr_t)(dst + j)) & 15) == 0)) {
                uint32_t wv[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * q]),
                                                                    __uint_as_float(r[j + 2 * q + 1]));
                    wv[q] = *reinterpret_cast<const uint32_t*>(&h2);
                }
                *reinterpret_cast<uint4*>(dst + j) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (col + e < N) dst[j + e] = __float2bfloat16_rn(__uint_as_float(r[j + e]));
            }
        }
    } else if (row < M) {
        float* dst = C + (size_t)row * ldc + col0;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const int col = col0 + j;
            if (col + 3 < N && ((((uintptr_t)dst) & 15) == 0)) {
                *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                                  __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (col + e < N) dst[j + e] = __uint_as_float(r[j + e]);
            }
        }
    }
}

// Progress of the two single-thread roles, kept in shared memory so that a CTA that gives up can tell which
// stages still have bulk copies in flight.
struct RoleProgress {
    int issued;    // stages the producer has armed and issued loads for
    int consumed;  // stages whose full barrier the MMA issuer has seen flip
    int failed;    // some wait of this CTA ran out
};

// Teardown after a wait ran out (called by one thread, after the block-wide barrier that follows the role
// loops): every stage that was armed but never consumed may still be the target of a bulk copy, and the CTA
// must not retire while one can land in its shared memory, so wait (bounded again) for those barriers.
__device__ __forceinline__ void drain_stages(const RoleProgress* pr, uint64_t* full, int stages, uint32_t limit) {
    for (int it = pr->consumed; it < pr->issued; ++it) mbar_wait(full + it % stages, (uint32_t)((it / stages) & 1), limit);
}

constexpr int kGemmStages = 3;
constexpr int kGemmBM = 128;
constexpr int kGemmBK = 64;  // bf16 elements: one 128-byte swizzle row

template <int BN>
struct GemmSmem {
    static constexpr int kA = kGemmBM * kGemmBK * 2;
    static constexpr int kB = BN * kGemmBK * 2;
    static constexpr int kStage = kA + kB;
    static constexpr int kBytes = kGemmStages * kStage + 1024 /* alignment slack */ + 256 /* barriers */;
};

// Stage of the NT kernel: with the hi/lo split one stage holds A_hi, A_lo, B_hi, B_lo of one K block, so
// the three products hi*hi + lo*hi + hi*lo reuse each tile from shared memory (two thirds of the
// L2 -> SM traffic of three separate passes).
template <int BN, bool SPLIT>
struct NtSmem {
    static constexpr int kA = kGemmBM * kGemmBK * 2;
    static constexpr int kB = BN * kGemmBK * 2;
    static constexpr int kStage = (SPLIT ? 2 : 1) * (kA + kB);
    static constexpr int kStagesRaw = (200 * 1024) / kStage;
    static constexpr int kStages = kStagesRaw > 4 ? 4 : (kStagesRaw < 2 ? 2 : kStagesRaw);
    static constexpr int kBytes = kStages * kStage + 1024 + 256;
};

template <int BN, bool SPLIT>
__global__ void __launch_bounds__(128)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                 const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                 float* __restrict__ C, int M, int N, int ldc, int k_blocks, int c_is_bf16, int* status) {
    using SM = NtSmem<BN, SPLIT>;
    constexpr int kStages = SM::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + kStages * SM::kStage);
    uint64_t* full = bars;                   // [stages] TMA -> MMA
    uint64_t* empty = bars + kStages;        // [stages] MMA -> TMA
    uint64_t* acc_ready = bars + 2 * kStages;
    uint64_t* drained = bars + 2 * kStages + 1;  // teardown only: the MMAs issued before giving up have finished
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kStages + 2);
    RoleProgress* progress = (RoleProgress*)(tmem_slot + 1);
    constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;  // power of two >= 32

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * kGemmBM, n0 = blockIdx.y * BN;
    const int total = k_blocks;
    const uint32_t limit = d_poll_limit;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        mbar_init(acc_ready, 1);
        mbar_init(drained, 1);
        progress->issued = progress->consumed = progress->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    bool ok = true;
    if (warp == 0 && lane == 0) {
        // ---- TMA producer: one K block per stage, all operand planes of it
        const int stop = d_withhold_from >= 0 ? min(total, d_withhold_from) : total;
        int it = 0;
        for (; it < stop && ok; ++it) {
            const int s = it % kStages, round = it / kStages;
            if (round > 0) ok = mbar_wait(empty + s, (round - 1) & 1, limit);
            if (!ok) break;
            uint8_t* st = smem + s * SM::kStage;
            mbar_expect_tx(full + s, SM::kStage);
            tma_load_2d(st, &map_a_hi, full + s, it * kGemmBK, m0);
            tma_load_2d(st + SM::kA, &map_b_hi, full + s, it * kGemmBK, n0);
            if (SPLIT) {
                tma_load_2d(st + SM::kA + SM::kB, &map_a_lo, full + s, it * kGemmBK, m0);
                tma_load_2d(st + 2 * SM::kA + SM::kB, &map_b_lo, full + s, it * kGemmBK, n0);
            }
        }
        progress->issued = it;
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer.  Instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major.
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                   ((uint32_t)(kGemmBM >> 4) << 24);
        int it = 0;
        for (; it < total && ok; ++it) {
            const int s = it % kStages, round = it / kStages;
            ok = mbar_wait(full + s, round & 1, limit);
            if (!ok) break;
            tc_fence_after();
            const uint32_t st = smem_u32(smem + s * SM::kStage);
            const uint64_t da_hi = umma_desc_k_sw128(st), db_hi = umma_desc_k_sw128(st + SM::kA);
            const uint64_t da_lo = umma_desc_k_sw128(st + SM::kA + SM::kB);
            const uint64_t db_lo = umma_desc_k_sw128(st + 2 * SM::kA + SM::kB);
#pragma unroll
            for (int k = 0; k < kGemmBK / 16; ++k) {
                // 16 bf16 = 32 bytes further along K inside the swizzle row: +2 in 16-byte units.
                tc_mma_bf16(tmem_base, da_hi + 2 * k, db_hi + 2 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
                if (SPLIT) {
                    tc_mma_bf16(tmem_base, da_lo + 2 * k, db_hi + 2 * k, idesc, 1u);
                    tc_mma_bf16(tmem_base, da_hi + 2 * k, db_lo + 2 * k, idesc, 1u);
                }
            }
            tc_commit(empty + s);  // arrives once the MMAs above have finished reading the stage
        }
        progress->consumed = it;
        if (ok) {
            tc_commit(acc_ready);
        } else {
            // giving up: tensor memory may only be released once the MMAs already issued have finished
            tc_commit(drained);
            mbar_wait(drained, 0, limit);
        }
    }
    if (!ok) {
        atomicExch(status, 1);
        progress->failed = 1;
    }

    // ---- epilogue: all four warps; warp w owns accumulator lanes [32w, 32w + 32).
    __syncwarp();
    // one decision per warp: the tcgen05.ld below is a warp-wide (.sync.aligned) instruction
    const bool ready = __all_sync(kFullMask, mbar_wait(acc_ready, 0, limit));
    if (!ready && lane == 0) {
        atomicExch(status, 2);
        progress->failed = 1;
    }
    tc_fence_after();
    if (ready) {
        const int row = m0 + warp * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r[32];
            tc_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
            store_acc_segment(r, row, M, N, n0 + c0, C, ldc, c_is_bf16);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && progress->failed) drain_stages(progress, full, kStages, limit);
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}


// Persistent form of the kernel above: one CTA per SM walks the output tiles, the accumulator is
// double-buffered in tensor memory (2 x BN columns), and the roles never meet inside a tile:
//   warp 0, one lane : TMA producer, runs ahead across tile boundaries (the stage ring never drains)
//   warp 1, one lane : MMA issuer, starts the next tile in the other accumulator as soon as that one is free
//   warps 2-5        : epilogue of the finished accumulator (warp w reads tensor-memory lanes
//                      [32 (w % 4), 32 (w % 4) + 32)), then hands the accumulator back
// so the pipeline fill and the epilogue of one tile overlap the main loop of its neighbors.
template <int BN, bool SPLIT>
__global__ void __launch_bounds__(192)
gemm_bf16_persistent_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                            const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                            float* __restrict__ C, int M, int N, int ldc, int k_blocks, int c_is_bf16, int n_tiles,
                            int num_tiles, int* status) {
    using SM = NtSmem<BN, SPLIT>;
    constexpr int kStages = SM::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + kStages * SM::kStage);
    uint64_t* full = bars;                       // [stages] TMA -> MMA
    uint64_t* empty = bars + kStages;            // [stages] MMA -> TMA
    uint64_t* acc_full = bars + 2 * kStages;     // [2] MMA -> epilogue
    uint64_t* acc_empty = bars + 2 * kStages + 2;  // [2] epilogue (4 warps) -> MMA
    uint64_t* drained = bars + 2 * kStages + 4;  // teardown only: the MMAs issued before giving up have finished
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kStages + 5);
    RoleProgress* progress = (RoleProgress*)(tmem_slot + 1);
    constexpr uint32_t kAccCols = BN < 32 ? 32 : BN;
    constexpr uint32_t kTmemCols = 2 * kAccCols;  // a power of two in [64, 512]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t limit = d_poll_limit;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full + a, 1);
            mbar_init(acc_empty + a, 4);
        }
        mbar_init(drained, 1);
        progress->issued = progress->consumed = progress->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    bool ok = true;
    if (warp == 0 && lane == 0) {
        int it = 0;
        const int withhold = d_withhold_from;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            const int m0 = (tile / n_tiles) * kGemmBM, n0 = (tile % n_tiles) * BN;
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                if (withhold >= 0 && it >= withhold) {  // test hook: nothing more is issued
                    ok = false;
                    break;
                }
                const int s = it % kStages, round = it / kStages;
                if (round > 0) ok = mbar_wait(empty + s, (round - 1) & 1, limit);
                if (!ok) break;
                uint8_t* st = smem + s * SM::kStage;
                mbar_expect_tx(full + s, SM::kStage);
                tma_load_2d(st, &map_a_hi, full + s, kb * kGemmBK, m0);
                tma_load_2d(st + SM::kA, &map_b_hi, full + s, kb * kGemmBK, n0);
                if (SPLIT) {
                    tma_load_2d(st + SM::kA + SM::kB, &map_a_lo, full + s, kb * kGemmBK, m0);
                    tma_load_2d(st + 2 * SM::kA + SM::kB, &map_b_lo, full + s, kb * kGemmBK, n0);
                }
            }
        }
        progress->issued = it;
        if (!ok) {
            atomicExch(status, 1);
            progress->failed = 1;
        }
    } else if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                   ((uint32_t)(kGemmBM >> 4) << 24);
        int it = 0, local = 0;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
            const int a = local & 1, use = local >> 1;
            // the first use of an accumulator finds its barrier in the initial phase and passes at once
            ok = mbar_wait(acc_empty + a, (uint32_t)((use & 1) ^ 1), limit);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + (uint32_t)a * kAccCols;
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                const int s = it % kStages, round = it / kStages;
                ok = mbar_wait(full + s, round & 1, limit);
                if (!ok) break;
                tc_fence_after();
                const uint32_t st = smem_u32(smem + s * SM::kStage);
                const uint64_t da_hi = umma_desc_k_sw128(st), db_hi = umma_desc_k_sw128(st + SM::kA);
                const uint64_t da_lo = umma_desc_k_sw128(st + SM::kA + SM::kB);
                const uint64_t db_lo = umma_desc_k_sw128(st + 2 * SM::kA + SM::kB);
#pragma unroll
                for (int k = 0; k < kGemmBK / 16; ++k) {
                    tc_mma_bf16(acc, da_hi + 2 * k, db_hi + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    if (SPLIT) {
                        tc_mma_bf16(acc, da_lo + 2 * k, db_hi + 2 * k, idesc, 1u);
                        tc_mma_bf16(acc, da_hi + 2 * k, db_lo + 2 * k, idesc, 1u);
                    }
                }
                tc_commit(empty + s);
            }
            if (ok) tc_commit(acc_full + a);
        }
        progress->consumed = it;
        if (!ok) {
            atomicExch(status, 1);
            progress->failed = 1;
            // tensor memory may only be released once the MMAs already issued have finished
            tc_commit(drained);
            mbar_wait(drained, 0, limit);
        }
    } else if (warp >= 2) {
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
            const int a = local & 1, use = local >> 1;
            const int m0 = (tile / n_tiles) * kGemmBM, n0 = (tile % n_tiles) * BN;
            // one decision per warp: the tcgen05.ld below is a warp-wide (.sync.aligned) instruction
            if (!__all_sync(kFullMask, mbar_wait(acc_full + a, (uint32_t)(use & 1), limit))) {
                if (lane == 0) {
                    atomicExch(status, 2);
                    progress->failed = 1;
                }
                break;
            }
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tc_ld_32x32(tmem_base + (uint32_t)a * kAccCols + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
                store_acc_segment(r, row, M, N, n0 + c0, C, ldc, c_is_bf16);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + a);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && progress->failed) drain_stages(progress, full, kStages, limit);
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// C[I, N] += A[rows, I]^T * B[rows, N]: both operands are row-major with the reduction index as
// the row, i.e. MN-major for the tensor core.  This is the weight gradient dW = P^T g
// (pccnn_lib_ops/pcconvs/kpconv.cu:90-93 of the reference).  grid = (I tiles, N tiles, splits):
// every CTA reduces its slab of rows in tensor memory and adds its tile to C with float
// reductions, so C must be zeroed by the caller.  Same roles and bounded waits as the kernel above.
template <int BN>
__global__ void __launch_bounds__(128)
gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
                    const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo,
                    float* __restrict__ C, int I, int N, int ldc, int k_blocks_total, int passes, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + kGemmStages * GemmSmem<BN>::kStage);
    uint64_t* full = bars;
    uint64_t* empty = bars + kGemmStages;
    uint64_t* acc_ready = bars + 2 * kGemmStages;
    uint64_t* drained = bars + 2 * kGemmStages + 1;  // teardown only: the MMAs issued before giving up have finished
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * kGemmStages + 2);
    RoleProgress* progress = (RoleProgress*)(tmem_slot + 1);
    constexpr uint32_t kTmemCols = BN;
    constexpr int kHalf = 64 * kGemmBK * 2;  // one 64-row x 64-column box: 8 KB

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i0 = blockIdx.x * kGemmBM, n0 = blockIdx.y * BN;
    // slab of 64-row blocks owned by this split
    const int per = (k_blocks_total + gridDim.z - 1) / gridDim.z;
    const int kb_begin = blockIdx.z * per;
    const int kb_end = min(k_blocks_total, kb_begin + per);
    const int k_blocks = kb_end - kb_begin;
    if (k_blocks <= 0) return;
    const int total = k_blocks * passes;
    const uint32_t limit = d_poll_limit;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGemmStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        mbar_init(acc_ready, 1);
        mbar_init(drained, 1);
        progress->issued = progress->consumed = progress->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    bool ok = true;
    if (warp == 0 && lane == 0) {
        const int stop = d_withhold_from >= 0 ? min(total, d_withhold_from) : total;
        int it = 0;
        for (; it < stop && ok; ++it) {
            const int s = it % kGemmStages, round = it / kGemmStages;
            if (round > 0) ok = mbar_wait(empty + s, (round - 1) & 1, limit);
            if (!ok) break;
            const int pass = it / k_blocks, kb = kb_begin + (it - pass * k_blocks);
            const CUtensorMap* ma = (pass == 1) ? &map_a_lo : &map_a_hi;
            const CUtensorMap* mb = (pass == 2) ? &map_b_lo : &map_b_hi;
            uint8_t* sa = smem + s * GemmSmem<BN>::kStage;
            mbar_expect_tx(full + s, GemmSmem<BN>::kStage);
            tma_load_2d(sa, ma, full + s, i0, kb * 64);
            tma_load_2d(sa + kHalf, ma, full + s, i0 + 64, kb * 64);
#pragma unroll
            for (int h = 0; h < BN / 64; ++h)
                tma_load_2d(sa + GemmSmem<BN>::kA + h * kHalf, mb, full + s, n0 + h * 64, kb * 64);
        }
        progress->issued = it;
    } else if (warp == 1 && lane == 0) {
        // fp32 accumulate, bf16 x bf16, both operands MN-major (bits 15 and 16).
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kGemmBM >> 4) << 24);
        int it = 0;
        for (; it < total && ok; ++it) {
            const int s = it % kGemmStages, round = it / kGemmStages;
            ok = mbar_wait(full + s, round & 1, limit);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * GemmSmem<BN>::kStage);
            const uint64_t da = umma_desc_mn_sw128(sa, kHalf), db = umma_desc_mn_sw128(sa + GemmSmem<BN>::kA, kHalf);
#pragma unroll
            for (int k = 0; k < 64 / 16; ++k) {
                // 16 reduction rows = 2048 bytes further: +128 in 16-byte units.
                tc_mma_bf16(tmem_base, da + 128 * k, db + 128 * k, idesc, (it > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit(empty + s);
        }
        progress->consumed = it;
        if (ok) {
            tc_commit(acc_ready);
        } else {
            // giving up: tensor memory may only be released once the MMAs already issued have finished
            tc_commit(drained);
            mbar_wait(drained, 0, limit);
        }
    }
    if (!ok) {
        atomicExch(status, 3);
        progress->failed = 1;
    }

    __syncwarp();
    // one decision per warp: the tcgen05.ld below is a warp-wide (.sync.aligned) instruction
    const bool ready = __all_sync(kFullMask, mbar_wait(acc_ready, 0, limit));
    if (!ready && lane == 0) {
        atomicExch(status, 4);
        progress->failed = 1;
    }
    tc_fence_after();
    if (ready) {
        const int row = i0 + warp * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t r[32];
            tc_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
            if (row < I) {
                float* dst = C + (size_t)row * ldc + n0 + c0;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (n0 + c0 + j < N) atomicAdd(dst + j, __uint_as_float(r[j]));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && progress->failed) drain_stages(progress, full, kGemmStages, limit);
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---- fp32 -> (hi, lo) bf16 split with zero padding ------------------------------------------
__global__ void __launch_bounds__(256)
split_bf16_kernel(int64_t rows, int cols, const float* __restrict__ src, int64_t ld_src, int ld_dst,
                  __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo) {
    const int64_t total = rows * ld_dst;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / ld_dst;
        const int c = (int)(i - r * ld_dst);
        const float v = (c < cols) ? src[r * ld_src + c] : 0.f;
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        hi[i] = h;
        if (lo) lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
    }
}

// Transposing variant: dst[c, r] = src[r, c]; dst rows (one per source column) padded to ld_dst.
__global__ void __launch_bounds__(256)
split_bf16_transpose_kernel(int rows, int cols, const float* __restrict__ src, int64_t ld_src, int ld_dst,
                            __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo) {
    const int64_t total = (int64_t)cols * ld_dst;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t c = i / ld_dst;
        const int r = (int)(i - c * ld_dst);
        const float v = (r < rows) ? src[(int64_t)r * ld_src + c] : 0.f;
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        hi[i] = h;
        if (lo) lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
    }
}

// dst[c, r] = src[r, c] for bf16 matrices; destination rows padded with zeros to ld_dst.
__global__ void __launch_bounds__(256)
transpose_bf16_kernel(int rows, int cols, const __nv_bfloat16* __restrict__ src, int64_t ld_src, int ld_dst,
                      __nv_bfloat16* __restrict__ dst) {
    const int64_t total = (int64_t)cols * ld_dst;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t c = i / ld_dst;
        const int r = (int)(i - c * ld_dst);
        dst[i] = (r < rows) ? src[(int64_t)r * ld_src + c] : __float2bfloat16_rn(0.f);
    }
}

// ---- host side ------------------------------------------------------------------------------
static uint32_t g_host_poll_limit = 1u << 21;  // host mirror of d_poll_limit for kernels of other translation units
uint32_t tensor_core_poll_limit() { return g_host_poll_limit; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// 2-D bf16 tensor [rows, ld] (ld elements per row, K contiguous), box = box_rows x 64, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t ld, int box_rows, int64_t cols = 0) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return PCCNN_ERR_CUDA;
    }
    if (((uintptr_t)base & 15) || (ld % 64)) {
        set_error("gemm operand must be 16-byte aligned with rows padded to 64 elements (ld = %lld)", (long long)ld);
        return PCCNN_ERR_INVALID;
    }
    cuuint64_t dims[2] = {(cuuint64_t)(cols > 0 && cols < ld ? cols : ld), (cuuint64_t)(rows > 0 ? rows : 1)};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)kGemmBK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with code %d (rows %lld, ld %lld, box %d)", (int)r, (long long)rows,
                  (long long)ld, box_rows);
        return PCCNN_ERR_CUDA;
    }
    return PCCNN_OK;
}

template <int BN, bool SPLIT>
static int launch_gemm_impl(const CUtensorMap& ma_hi, const CUtensorMap& ma_lo, const CUtensorMap& mb_hi,
                            const CUtensorMap& mb_lo, float* C, int64_t M, int N, int K_padded, int ldc, int c_is_bf16,
                            int* status, cudaStream_t s) {
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<BN, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        NtSmem<BN, SPLIT>::kBytes);
        if (attr_err == cudaSuccess)
            attr_err = cudaFuncSetAttribute(gemm_bf16_persistent_kernel<BN, SPLIT>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, NtSmem<BN, SPLIT>::kBytes);
    });
    PCCNN_CUDA(attr_err);
    const int m_tiles = (int)((M + kGemmBM - 1) / kGemmBM), n_tiles = (N + BN - 1) / BN;
    const long long num_tiles = (long long)m_tiles * n_tiles;
    if (num_tiles > sm_count() && num_tiles < 0x7fffffffLL) {
        // more tiles than SMs: one persistent CTA per SM, fill and epilogue hidden behind neighboring tiles
        gemm_bf16_persistent_kernel<BN, SPLIT><<<sm_count(), 192, NtSmem<BN, SPLIT>::kBytes, s>>>(
            ma_hi, ma_lo, mb_hi, mb_lo, C, (int)M, N, ldc, K_padded / kGemmBK, c_is_bf16, n_tiles, (int)num_tiles, status);
    } else {
        dim3 grid((unsigned)m_tiles, (unsigned)n_tiles);
        gemm_bf16_kernel<BN, SPLIT><<<grid, 128, NtSmem<BN, SPLIT>::kBytes, s>>>(ma_hi, ma_lo, mb_hi, mb_lo, C, (int)M, N, ldc,
                                                                              K_padded / kGemmBK, c_is_bf16, status);
    }
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

template <int BN>
static int launch_gemm(const GemmOperand& a, const GemmOperand& b, float* C, int64_t M, int N, int K_padded, int ldc,
                       int c_is_bf16, int* status, cudaStream_t s) {
    CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo;
    const bool split = a.lo && b.lo;
    if (int rc = make_map(&ma_hi, a.hi, M, a.ld, kGemmBM, a.cols)) return rc;
    if (int rc = make_map(&ma_lo, split ? a.lo : a.hi, M, a.ld, kGemmBM, a.cols)) return rc;
    if (int rc = make_map(&mb_hi, b.hi, N, b.ld, BN, b.cols)) return rc;
    if (int rc = make_map(&mb_lo, split ? b.lo : b.hi, N, b.ld, BN, b.cols)) return rc;
    if (split) return launch_gemm_impl<BN, true>(ma_hi, ma_lo, mb_hi, mb_lo, C, M, N, K_padded, ldc, c_is_bf16, status, s);
    return launch_gemm_impl<BN, false>(ma_hi, ma_lo, mb_hi, mb_lo, C, M, N, K_padded, ldc, c_is_bf16, status, s);
}

int gemm_bf16_nt(const GemmOperand& a, const GemmOperand& b, float* C, int64_t M, int N, int K_padded, int ldc,
                 int* status, cudaStream_t s, int c_is_bf16) {
    PCCNN_CHECK_ARG(M >= 0 && M < 0x7fffffffLL && N > 0 && K_padded > 0 && K_padded % kGemmBK == 0,
                    "gemm: bad shape M=%lld N=%d K=%d", (long long)M, N, K_padded);
    PCCNN_CHECK_ARG(a.ld >= K_padded && b.ld >= K_padded, "gemm: leading dimensions smaller than K");
    if (M == 0) return PCCNN_OK;
    if (N <= 16) return launch_gemm<16>(a, b, C, M, N, K_padded, ldc, c_is_bf16, status, s);
    if (N <= 32) return launch_gemm<32>(a, b, C, M, N, K_padded, ldc, c_is_bf16, status, s);
    if (N <= 64) return launch_gemm<64>(a, b, C, M, N, K_padded, ldc, c_is_bf16, status, s);
    if (N <= 128) return launch_gemm<128>(a, b, C, M, N, K_padded, ldc, c_is_bf16, status, s);
    return launch_gemm<256>(a, b, C, M, N, K_padded, ldc, c_is_bf16, status, s);
}

template <int BN>
static int launch_gemm_tn(const GemmOperand& a, const GemmOperand& b, float* C, int64_t rows, int I, int N, int ldc,
                          int* status, cudaStream_t s) {
    CUtensorMap ma_hi, ma_lo, mb_hi, mb_lo;
    const int passes = (a.lo && b.lo) ? 3 : 1;
    if (int rc = make_map(&ma_hi, a.hi, rows, a.ld, 64, a.cols)) return rc;
    if (int rc = make_map(&ma_lo, passes == 3 ? a.lo : a.hi, rows, a.ld, 64, a.cols)) return rc;
    if (int rc = make_map(&mb_hi, b.hi, rows, b.ld, 64, b.cols)) return rc;
    if (int rc = make_map(&mb_lo, passes == 3 ? b.lo : b.hi, rows, b.ld, 64, b.cols)) return rc;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(gemm_bf16_tn_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        GemmSmem<BN>::kBytes);
    });
    PCCNN_CUDA(attr_err);
    const int k_blocks = (int)((rows + 63) / 64);
    const int tiles = ((I + kGemmBM - 1) / kGemmBM) * ((N + BN - 1) / BN);
    int splits = (2 * sm_count() + tiles - 1) / tiles;  // about two CTAs per SM in total
    if (splits > k_blocks) splits = k_blocks;
    if (splits < 1) splits = 1;
    dim3 grid((unsigned)((I + kGemmBM - 1) / kGemmBM), (unsigned)((N + BN - 1) / BN), (unsigned)splits);
    gemm_bf16_tn_kernel<BN><<<grid, 128, GemmSmem<BN>::kBytes, s>>>(ma_hi, ma_lo, mb_hi, mb_lo, C, I, N, ldc, k_blocks,
                                                                  passes, status);
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

int gemm_bf16_tn_accumulate(const GemmOperand& a, const GemmOperand& b, float* C, int64_t rows, int I, int N, int ldc,
                            int* status, cudaStream_t s) {
    PCCNN_CHECK_ARG(rows >= 0 && rows < 0x7fffffffLL && I > 0 && N > 0, "gemm_tn: bad shape");
    PCCNN_CHECK_ARG(a.ld >= (I + 63) / 64 * 64 && b.ld >= (N + 63) / 64 * 64,
                    "gemm_tn: operand rows must be padded to a multiple of 64 elements");
    if (rows == 0) return PCCNN_OK;
    if (N <= 64) return launch_gemm_tn<64>(a, b, C, rows, I, N, ldc, status, s);
    if (N <= 128) return launch_gemm_tn<128>(a, b, C, rows, I, N, ldc, status, s);
    return launch_gemm_tn<256>(a, b, C, rows, I, N, ldc, status, s);
}

int transpose_bf16(int rows, int cols, const void* src, int64_t ld_src, int ld_dst, void* dst, cudaStream_t s) {
    if (rows == 0 || cols == 0) return PCCNN_OK;
    transpose_bf16_kernel<<<grid_for((int64_t)cols * ld_dst, 256, 8), 256, 0, s>>>(
        rows, cols, (const __nv_bfloat16*)src, ld_src, ld_dst, (__nv_bfloat16*)dst);
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

int split_bf16(int64_t rows, int cols, const float* src, int64_t ld_src, int ld_dst, void* hi, void* lo,
               cudaStream_t s) {
    if (rows == 0) return PCCNN_OK;
    split_bf16_kernel<<<grid_for(rows * ld_dst, 256, 8), 256, 0, s>>>(rows, cols, src, ld_src, ld_dst,
                                                                    (__nv_bfloat16*)hi, (__nv_bfloat16*)lo);
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

int split_bf16_transpose(int rows, int cols, const float* src, int64_t ld_src, int ld_dst, void* hi, void* lo,
                         cudaStream_t s) {
    if (rows == 0 || cols == 0) return PCCNN_OK;
    split_bf16_transpose_kernel<<<grid_for((int64_t)cols * ld_dst, 256, 8), 256, 0, s>>>(
        rows, cols, src, ld_src, ld_dst, (__nv_bfloat16*)hi, (__nv_bfloat16*)lo);
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

}  // namespace pccnn

using namespace pccnn;

extern "C" {

int pccnn_gemm_set_test_hooks(int poll_limit, int withhold_from) {
    const uint32_t limit = poll_limit > 0 ? (uint32_t)poll_limit : (1u << 21);
    g_host_poll_limit = limit;
    const int withhold = withhold_from >= 0 ? withhold_from : -1;
    PCCNN_CUDA(cudaMemcpyToSymbol(d_poll_limit, &limit, sizeof(limit)));
    PCCNN_CUDA(cudaMemcpyToSymbol(d_withhold_from, &withhold, sizeof(withhold)));
    return PCCNN_OK;
}

size_t pccnn_gemm_workspace_bytes(int64_t M, int N, int K) {
    const int64_t kp = (K + 63) / 64 * 64;
    return (size_t)(align_up((size_t)M * kp * 2) * 2 + align_up((size_t)N * kp * 2) * 2 + 256);
}

int pccnn_gemm_f32(int64_t M, int N, int K, const float* A, int64_t lda, const float* B, int64_t ldb, float* C,
                   int64_t ldc, int split, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(M >= 0 && N > 0 && K > 0, "gemm_f32: bad shape");
    if (M == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(A && B && C, "gemm_f32: null pointer");
    if (!workspace || workspace_bytes < pccnn_gemm_workspace_bytes(M, N, K)) {
        set_error("gemm_f32: workspace of %zu bytes, need %zu", workspace_bytes, pccnn_gemm_workspace_bytes(M, N, K));
        return PCCNN_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int kp = (K + 63) / 64 * 64;
    char* ws = (char*)workspace;
    const size_t a_bytes = align_up((size_t)M * kp * 2), b_bytes = align_up((size_t)N * kp * 2);
    GemmOperand a{ws, split ? ws + a_bytes : nullptr, kp};
    GemmOperand b{ws + 2 * a_bytes, split ? ws + 2 * a_bytes + b_bytes : nullptr, kp};
    int* status = (int*)(ws + 2 * a_bytes + 2 * b_bytes);
    PCCNN_CUDA(cudaMemsetAsync(status, 0, 4, s));
    if (int rc = split_bf16(M, K, A, lda, kp, a.hi, a.lo, s)) return rc;
    if (int rc = split_bf16(N, K, B, ldb, kp, b.hi, b.lo, s)) return rc;
    if (int rc = gemm_bf16_nt(a, b, C, M, N, kp, (int)ldc, status, s)) return rc;
    int host_status = 0;
    PCCNN_CUDA(cudaMemcpyAsync(&host_status, status, 4, cudaMemcpyDeviceToHost, s));
    PCCNN_CUDA(cudaStreamSynchronize(s));
    if (host_status != 0) {
        set_error("gemm_f32: a bounded wait inside the tensor-core kernel ran out (status %d)", host_status);
        return PCCNN_ERR_DEVICE;
    }
    return PCCNN_OK;
}

int pccnn_gemm_bf16(int64_t M, int N, int K, const void* a_hi, const void* a_lo, int64_t lda, const void* b_hi,
                    const void* b_lo, int64_t ldb, float* C, int64_t ldc, int* status_dev, void* stream) {
    PCCNN_CHECK_ARG(a_hi && b_hi && C && status_dev, "gemm_bf16: null pointer");
    PCCNN_CHECK_ARG((a_lo == nullptr) == (b_lo == nullptr), "gemm_bf16: give the lo parts of both operands or of neither");
    GemmOperand a{const_cast<void*>(a_hi), const_cast<void*>(a_lo), lda};
    GemmOperand b{const_cast<void*>(b_hi), const_cast<void*>(b_lo), ldb};
    return gemm_bf16_nt(a, b, C, M, N, K, (int)ldc, status_dev, (cudaStream_t)stream);
}

size_t pccnn_gemm_tn_workspace_bytes(int64_t rows, int I, int N) {
    const int64_t ip = (I + 63) / 64 * 64, np_ = (N + 63) / 64 * 64;
    return (size_t)(align_up((size_t)rows * ip * 2) * 2 + align_up((size_t)rows * np_ * 2) * 2 + 256);
}

int pccnn_gemm_tn_f32(int64_t rows, int I, int N, const float* A, int64_t lda, const float* B, int64_t ldb, float* C,
                      int64_t ldc, int split, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(rows >= 0 && I > 0 && N > 0, "gemm_tn_f32: bad shape");
    PCCNN_CHECK_ARG(A && B && C, "gemm_tn_f32: null pointer");
    if (!workspace || workspace_bytes < pccnn_gemm_tn_workspace_bytes(rows, I, N)) {
        set_error("gemm_tn_f32: workspace too small");
        return PCCNN_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int ip = (I + 63) / 64 * 64, np_ = (N + 63) / 64 * 64;
    char* ws = (char*)workspace;
    const size_t a_bytes = align_up((size_t)rows * ip * 2), b_bytes = align_up((size_t)rows * np_ * 2);
    GemmOperand a{ws, split ? ws + a_bytes : nullptr, ip};
    GemmOperand b{ws + 2 * a_bytes, split ? ws + 2 * a_bytes + b_bytes : nullptr, np_};
    int* status = (int*)(ws + 2 * a_bytes + 2 * b_bytes);
    PCCNN_CUDA(cudaMemsetAsync(status, 0, 4, s));
    for (int64_t r = 0; r < I; ++r) PCCNN_CUDA(cudaMemsetAsync(C + r * ldc, 0, (size_t)N * 4, s));
    if (int rc = split_bf16(rows, I, A, lda, ip, a.hi, a.lo, s)) return rc;
    if (int rc = split_bf16(rows, N, B, ldb, np_, b.hi, b.lo, s)) return rc;
    if (int rc = gemm_bf16_tn_accumulate(a, b, C, rows, I, N, (int)ldc, status, s)) return rc;
    int host_status = 0;
    PCCNN_CUDA(cudaMemcpyAsync(&host_status, status, 4, cudaMemcpyDeviceToHost, s));
    PCCNN_CUDA(cudaStreamSynchronize(s));
    if (host_status != 0) {
        set_error("gemm_tn_f32: a bounded wait inside the tensor-core kernel ran out (status %d)", host_status);
        return PCCNN_ERR_DEVICE;
    }
    return PCCNN_OK;
}

}  // extern "C"
