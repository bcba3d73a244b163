// Pair-level contractions of the convolutions on the tensor cores (3-D points).
//
// The projection P[m, c, k] = sum_t F[n0(t), c] b[t, k] of the reference (pcconvs/shared/feat_basis_proj.cu:30-129
// of phermosilla/pccnn_lib) and the two contractions of its backward (feat_basis_proj_grads.cu:32-154)
//     dF[n0(t), c] += sum_k dP[m, c, k] b[t, k]          db[t, k] = sum_c dP[m, c, k] F[n0(t), c]
// are, per sample, small matrix products over the sample's neighbors.  The kernels here run them with tcgen05.mma:
// a CTA takes one sample at a time, its threads gather the neighbors' feature rows (once, as bf16 hi + lo planes) and
// evaluate the basis into 128-byte-swizzled shared-memory tiles, one thread issues the MMAs into tensor memory,
// and all threads read the result back (tcgen05.ld) for the epilogue.  Compared with the CUDA-core kernels of
// conv_impl.cuh the arithmetic per pair drops from ~70 (forward) / ~230 (backward) warp instructions to the few
// that move the pair's data.
//
// Shared-memory tiles (every operand is a K-major or MN-major SW128 tile, the layouts gemm.cu already uses):
//   F   [128 neighbors x 128 channels]  two 64-channel blocks of [128 rows x 128 B], hi and lo planes.
//       forward:  A operand, MN-major (M = channel, K = neighbor);  backward db: A operand, K-major (M = neighbor,
//       K = channel) -- the same bytes, two descriptor views.
//   BT  [NB basis x 128 neighbors]      forward B operand, K-major (N = basis, K = neighbor).
//   BM  [128 neighbors x 64 (NB used)]  backward dF A operand, K-major (M = neighbor, K = basis), rows padded to 128 B.
//   GP  [NB basis x 128 channels]       backward db B operand, K-major (N = basis, K = channel).
//   GQ  [128 channels x 64 (NB used)]   backward dF B operand, K-major (N = channel, K = basis), rows padded to 128 B.
// fp32 accuracy comes from the hi/lo split of both factors (three MMAs per product, lo * lo dropped).
#pragma once

#include <cuda_bf16.h>

#include <mutex>

#include "common.cuh"
#include "stencil.cuh"
#include "tc_ptx.cuh"

namespace pccnn {

constexpr int kTcRows = 128;  // neighbors per pass of a sample
constexpr int kTcChan = 128;  // channels per pass

__device__ __forceinline__ uint32_t pack_bf16x2(__nv_bfloat16 a, __nv_bfloat16 b) {
    return (uint32_t)__bfloat16_as_ushort(a) | ((uint32_t)__bfloat16_as_ushort(b) << 16);
}

// hi / lo bf16 parts of four floats, packed as two 32-bit words each
__device__ __forceinline__ void split4(const float (&v)[4], uint2& hi, uint2& lo) {
    __nv_bfloat16 h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        h[i] = __float2bfloat16_rn(v[i]);
        l[i] = __float2bfloat16_rn(v[i] - __bfloat162float(h[i]));
    }
    hi = make_uint2(pack_bf16x2(h[0], h[1]), pack_bf16x2(h[2], h[3]));
    lo = make_uint2(pack_bf16x2(l[0], l[1]), pack_bf16x2(l[2], l[3]));
}

// Features reach the pair kernels as bf16 planes (hi, and lo for fp32 inputs) with rows padded to a multiple of 8
// channels, so that a neighbor's row is a sequence of 16-byte chunks that can be copied without passing through
// registers.  fp32 features are split once per operator call (split_features below); bf16 features are used as they are.
struct FeaturePlanes {
    const __nv_bfloat16* hi;
    const __nv_bfloat16* lo;  // null: single plane
    int ld;                   // elements per row, a multiple of 8
};

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, bool valid) {
    // 16 bytes global -> shared without registers; src-size 0 writes zeros instead
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Starts the copies of the feature rows of the staged neighbors (s_n0[0 .. rows), -1 = no neighbor) for the channels
// [cb, cb + 128) into the F tile: warp w takes rows w, w + 4, ...; with two planes lanes 0-15 copy the 16 chunks of
// the hi plane and lanes 16-31 those of the lo plane (one warp instruction per row); with one plane the two half
// warps take two rows (NW = warps of the CTA).  Chunks past the row's end and rows without a neighbor are zero-filled.  Asynchronous: the
// caller waits (cp_async_wait_all) before the tile is used.
template <bool SPLIT_F, int NW = 4, bool HALF = false>
__device__ __forceinline__ void gather_features_async(uint32_t f_hi, uint32_t f_lo, const int* s_n0, int rows,
                                                      const FeaturePlanes& f, int cb) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunk = lane & 15;       // 8 channels
    if (HALF && chunk >= 8) return;    // a plane of one 64-channel block: nothing to copy (or to clear) behind it
    const int c = cb + 8 * chunk;
    const uint32_t in_tile = (uint32_t)(chunk >> 3) * (kTcRows * 128);
    if (SPLIT_F) {
        const __nv_bfloat16* plane = (lane < 16) ? f.hi : f.lo;
        const uint32_t tile = (lane < 16) ? f_hi : f_lo;
        for (int r = warp; r < rows; r += NW) {
            const int n0 = s_n0[r];
            const bool valid = n0 >= 0 && c < f.ld;
            cp_async_16(tile + in_tile + sw128_offset(r, chunk & 7), plane + (valid ? (int64_t)n0 * f.ld + c : 0), valid);
        }
    } else {
        for (int r = 2 * warp + (lane >> 4); r < rows; r += 2 * NW) {
            const int n0 = s_n0[r];
            const bool valid = n0 >= 0 && c < f.ld;
            cp_async_16(f_hi + in_tile + sw128_offset(r, chunk & 7), f.hi + (valid ? (int64_t)n0 * f.ld + c : 0), valid);
        }
    }
}

// fp32 [rows, cin] -> bf16 hi / lo planes [rows, ld] (ld = cin rounded up to 8, zero padded)
static __global__ void __launch_bounds__(256)
split_features_kernel(int64_t rows, int cin, int ld, const float* __restrict__ src, __nv_bfloat16* __restrict__ hi,
                      __nv_bfloat16* __restrict__ lo) {
    const int64_t total = rows * (ld / 8);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / (ld / 8);
        const int c = (int)(i - r * (ld / 8)) * 8;
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = (c + e < cin) ? __ldg(src + r * cin + c + e) : 0.f;
        uint32_t hw[4], lw[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
            const __nv_bfloat162 l2 = __floats2bfloat162_rn(v[2 * q] - __low2float(h2), v[2 * q + 1] - __high2float(h2));
            hw[q] = *reinterpret_cast<const uint32_t*>(&h2);
            lw[q] = *reinterpret_cast<const uint32_t*>(&l2);
        }
        *reinterpret_cast<uint4*>(hi + r * ld + c) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        *reinterpret_cast<uint4*>(lo + r * ld + c) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
    }
}

static int split_features(int64_t rows, int cin, const float* src, void* hi, void* lo, cudaStream_t s) {
    if (rows == 0) return PCCNN_OK;
    const int ld = (cin + 7) / 8 * 8;
    split_features_kernel<<<grid_for(rows * (ld / 8), 256, 8), 256, 0, s>>>(rows, cin, ld, src, (__nv_bfloat16*)hi,
                                                                            (__nv_bfloat16*)lo);
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

// K entries of channel c of a P row (bf16 hi [+ lo] planes): 128-bit stores when the K values of a channel are
// 16-byte aligned, element stores otherwise.
template <int NB>
__device__ __forceinline__ void store_p_row(const float (&acc)[NB], int c, int cin, int K, __nv_bfloat16* __restrict__ p_hi,
                                            __nv_bfloat16* __restrict__ p_lo, size_t row) {
    if (c >= cin) return;
    if (K == NB) {
#pragma unroll
        for (int k = 0; k < NB; k += 8) {
            uint32_t hw[4], lw[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float v0 = acc[k + 2 * q], v1 = acc[k + 2 * q + 1];
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(v0, v1);
                const __nv_bfloat162 l2 = __floats2bfloat162_rn(v0 - __low2float(h2), v1 - __high2float(h2));
                hw[q] = *reinterpret_cast<const uint32_t*>(&h2);
                lw[q] = *reinterpret_cast<const uint32_t*>(&l2);
            }
            *reinterpret_cast<uint4*>(p_hi + row + (size_t)c * K + k) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            if (p_lo) *reinterpret_cast<uint4*>(p_lo + row + (size_t)c * K + k) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
        }
    } else {
#pragma unroll
        for (int k = 0; k < NB; ++k) {
            if (k < K) {
                const __nv_bfloat16 h = __float2bfloat16_rn(acc[k]);
                p_hi[row + (size_t)c * K + k] = h;
                if (p_lo) p_lo[row + (size_t)c * K + k] = __float2bfloat16_rn(acc[k] - __bfloat162float(h));
            }
        }
    }
}

// SPLIT_F: the features come as two bf16 planes (fp32 inputs); with bf16 inputs there is no lo plane and the CTA is
// 32 KB smaller, so that five instead of three fit an SM.
// HALF: at most 64 input channels, so a plane of the F tile holds one 64-channel block instead of two and the
// products run with M = 64 (their 64 accumulator rows lie in lanes 0-15 of each quarter of the tensor memory).
template <int NB, bool SPLIT_F, bool HALF = false>
struct TcForwardSmem {
    static constexpr int kBlock = kTcRows * 128;          // one 64-channel block of a plane: 16 KB
    static constexpr int kF = (HALF ? 1 : 2) * kBlock;    // one plane of the F tile
    static constexpr int kBT = 2 * NB * 128;      // one plane of the BT tile: two 64-neighbor blocks of [NB x 128 B]
    static constexpr int kFPlanes = SPLIT_F ? 2 : 1;
    static constexpr int kFHi = 0, kFLo = SPLIT_F ? kF : 0, kBTHi = kFPlanes * kF, kBTLo = kBTHi + kBT;
    static constexpr int kTiles = kFPlanes * kF + 2 * kBT;
    static constexpr int kMisc = 2048;  // barrier, tensor-memory slot, neighbor ids, basis parameters
    static constexpr int kBytes = kTiles + kMisc;
    static constexpr int kGridBytes = kTiles + 2688;  // list-free variant: + candidate ranges and the hit queue
};

#ifdef PCCNN_TC_PROFILE
static __device__ long long g_tc_prof[16];
#define TC_PROF(i) do { if (blockIdx.x == 0 && tid == 0) { long long now_ = clock64(); prof_[i] += now_ - last_; last_ = now_; } } while (0)
#else
#define TC_PROF(i) do {} while (0)
#endif

// P rows (bf16 hi [+ lo]) of the samples [m_begin, m_end).  One CTA = one sample at a time.
template <int NB, class BASIS, class ARGS, bool SPLIT_F, bool HALF>
__global__ void __launch_bounds__(128)
project_tc_kernel(ARGS args, int K, const float* __restrict__ pts, FeaturePlanes feats, int cin,
                  const float* __restrict__ samples, const int2* __restrict__ neighbors,
                  const int32_t* __restrict__ start_ids, const float* __restrict__ radii, int m_begin, int m_end,
                  __nv_bfloat16* __restrict__ p_hi, __nv_bfloat16* __restrict__ p_lo, int ld_p, uint32_t poll_limit,
                  int* __restrict__ status) {
    using SM = TcForwardSmem<NB, SPLIT_F, HALF>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];  // the swizzled tiles need 1024-byte alignment
    uint8_t* smem = smem_raw;
    uint8_t* misc = smem + SM::kTiles;
    uint64_t* bar = (uint64_t*)misc;
    uint32_t* tmem_slot = (uint32_t*)(misc + 8);
    int* s_fail = (int*)(misc + 12);
    int* s_n0 = (int*)(misc + 64);              // [128]
    float* s_params = (float*)(misc + 64 + 512);  // up to 256 floats
    static_assert(BASIS::kParamFloats <= 256, "basis parameters do not fit the shared-memory slot");
    constexpr uint32_t kTmemCols = NB < 32 ? 32 : NB;

    const int tid = threadIdx.x, warp = tid >> 5;
    if (tid == 0) {
        mbar_init(bar, 1);
        *s_fail = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    BASIS::load_params(s_params, args, K);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    float inv[3];
#pragma unroll
    for (int d = 0; d < 3; ++d) inv[d] = BASIS::kUsesOffset ? __frcp_rn(__ldg(radii + d)) : 0.f;
    const int inner = cin * K;
    const uint32_t f_hi = smem_u32(smem + SM::kFHi), f_lo = smem_u32(smem + SM::kFLo);
    const uint32_t bt_hi = smem_u32(smem + SM::kBTHi), bt_lo = smem_u32(smem + SM::kBTLo);
    // fp32 accumulate, bf16 x bf16, A MN-major (bit 15), B K-major, N = NB, M = 128
    // (M = 64 with one channel block per plane)
    constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(NB >> 3) << 17) |
                               ((uint32_t)((HALF ? 64 : 128) >> 4) << 24);
    uint32_t parity = 0;
    bool failed = false;

    // The work of this CTA is a flat sequence of passes (sample, channel block, 128 neighbors), run as a software
    // pipeline: the loads a pass depends on (the sample's range, the neighbor ids, the neighbors' coordinates) are
    // issued one pass ahead, and the epilogue of a finished (sample, channel block) runs while the feature rows of
    // the next pass are being copied.
    struct Sample {
        int m, lo, hi;
        float s[3];
    };
    auto load_sample = [&](int m) {
        Sample q;
        q.m = m;
        q.lo = q.hi = 0;
        q.s[0] = q.s[1] = q.s[2] = 0.f;
        if (m < m_end) {
            q.lo = (m > 0) ? __ldg(start_ids + m - 1) : 0;
            q.hi = __ldg(start_ids + m);
#pragma unroll
            for (int d = 0; d < 3; ++d) q.s[d] = BASIS::kUsesOffset ? __ldg(samples + (int64_t)m * 3 + d) : 0.f;
        }
        return q;
    };
    auto load_id = [&](bool valid, int t0, int hi) {
        return (valid && t0 + tid < hi) ? __ldg(&neighbors[t0 + tid]).x : -1;
    };
    auto load_point = [&](int n0, float (&q)[3]) {
#pragma unroll
        for (int x = 0; x < 3; ++x) q[x] = (BASIS::kUsesOffset && n0 >= 0) ? __ldg(pts + (int64_t)n0 * 3 + x) : 0.f;
    };

    Sample cur = load_sample(m_begin + blockIdx.x);
    Sample ahead = load_sample(cur.m + gridDim.x);  // its loads are in flight while `cur` is processed
    int cb = 0, t0 = cur.lo;
    bool cur_valid = cur.m < m_end;
    int n0 = load_id(cur_valid, t0, cur.hi);
    float pt[3];
    load_point(n0, pt);
    // the (sample, channel block) whose accumulator waits for its epilogue
    bool epi = false, epi_nonempty = false;
    int epi_m = 0, epi_cb = 0;

#ifdef PCCNN_TC_PROFILE
    long long prof_[8] = {0, 0, 0, 0, 0, 0, 0, 0}, last_ = clock64();
#endif
    while ((cur_valid || epi) && !failed) {
        const int cnt = cur_valid ? min(kTcRows, cur.hi - t0) : 0;
        const int rows = (cnt + 15) & ~15;
        s_n0[tid] = n0;
        __syncthreads();
        TC_PROF(0);
        if (cnt > 0) gather_features_async<SPLIT_F, 4, HALF>(f_hi, f_lo, s_n0, rows, feats, cb);
        TC_PROF(1);

        // ---- epilogue of the previous (sample, channel block): thread = channel, NB columns -> K entries of the P row
        if (epi) {
            tc_fence_after();
            const size_t row = (size_t)(epi_m - m_begin) * ld_p;
            float acc[NB];
            if (!epi_nonempty) {  // no neighbor at all: the accumulator was never written
#pragma unroll
                for (int k = 0; k < NB; ++k) acc[k] = 0.f;
            } else {
#pragma unroll
                for (int k0 = 0; k0 < NB; k0 += 16) {
                    uint32_t r[16];
                    tc_ld_32x16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)k0, r);
#pragma unroll
                    for (int k = 0; k < 16; ++k) acc[k0 + k] = __uint_as_float(r[k]);
                }
            }
            if (HALF) {  // 64 accumulator rows: channel 16 w + l is in lane l < 16 of warp w's quarter
                if ((tid & 31) < 16) store_p_row<NB>(acc, epi_cb + 16 * warp + (tid & 31), cin, K, p_hi, p_lo, row);
            } else {
                store_p_row<NB>(acc, epi_cb + tid, cin, K, p_hi, p_lo, row);
            }
            if (epi_cb + kTcChan >= cin) {  // last channel block: the padding columns feed the contraction too
                for (int c = inner + tid; c < ld_p; c += 128) {
                    p_hi[row + c] = __float2bfloat16_rn(0.f);
                    if (p_lo) p_lo[row + c] = __float2bfloat16_rn(0.f);
                }
            }
            epi = false;
        }
        TC_PROF(2);

        // ---- the pass after this one, and its first loads
        Sample nxt = cur;
        int nxt_cb = cb, nxt_t0 = t0 + kTcRows;
        bool nxt_valid = cur_valid;
        const bool last_of_block = cur_valid && nxt_t0 >= cur.hi;
        if (last_of_block) {
            nxt_cb = cb + kTcChan;
            nxt_t0 = cur.lo;
            if (nxt_cb >= cin) {
                nxt = ahead;
                nxt_cb = 0;
                nxt_t0 = nxt.lo;
                nxt_valid = nxt.m < m_end;
                ahead = load_sample(nxt.m + gridDim.x);
            }
        }
        const int n0_next = load_id(nxt_valid, nxt_t0, nxt.hi);

        // ---- lanes as neighbors, while the copies are in flight: offset, basis, BT column of pair t0 + tid
        if (cnt > 0) {
            float b[NB];
            if (tid < cnt) {
                float d[3];
#pragma unroll
                for (int x = 0; x < 3; ++x) d[x] = (pt[x] - cur.s[x]) * inv[x];
                BASIS::eval(s_params, args, K, d, n0, t0 + tid, cur.m, b);
            } else {
#pragma unroll
                for (int k = 0; k < NB; ++k) b[k] = 0.f;
            }
            if (tid < rows) {
                uint8_t* base_hi = smem + SM::kBTHi + (tid >> 6) * (NB * 128) + (tid & 7) * 2;
                uint8_t* base_lo = smem + SM::kBTLo + (tid >> 6) * (NB * 128) + (tid & 7) * 2;
                const int chunk = (tid & 63) >> 3;
#pragma unroll
                for (int k = 0; k < NB; ++k) {
                    const __nv_bfloat16 h = __float2bfloat16_rn(b[k]);
                    const uint32_t off = sw128_offset(k, chunk);
                    *reinterpret_cast<__nv_bfloat16*>(base_hi + off) = h;
                    *reinterpret_cast<__nv_bfloat16*>(base_lo + off) = __float2bfloat16_rn(b[k] - __bfloat162float(h));
                }
            }
        }
        TC_PROF(3);
        cp_async_wait_all();
        fence_smem_to_async_proxy();
        tc_fence_before();
        __syncthreads();
        TC_PROF(4);
        if (cnt > 0 && tid == 0) {
            tc_fence_after();
            const bool first = t0 == cur.lo;
            for (int kb = 0; kb < rows / 16; ++kb) {
                // A: 16 neighbor rows further = 2048 bytes = +128 in 16-byte units; the two 64-channel blocks
                // are 16 KB apart (leading byte offset).  B: 64-neighbor block kb / 4, 16 neighbors = +2.
                const uint64_t a_hi = umma_desc_mn_sw128(f_hi, kTcRows * 128) + 128ull * kb;
                const uint64_t b_off = (uint64_t)(kb >> 2) * ((NB * 128) >> 4) + 2ull * (kb & 3);
                const uint64_t b_hi = umma_desc_k_sw128(bt_hi) + b_off, b_lo = umma_desc_k_sw128(bt_lo) + b_off;
                tc_mma_bf16(tmem_base, a_hi, b_hi, idesc, (!first || kb > 0) ? 1u : 0u);
                tc_mma_bf16(tmem_base, a_hi, b_lo, idesc, 1u);
                if (SPLIT_F) {
                    const uint64_t a_lo = umma_desc_mn_sw128(f_lo, kTcRows * 128) + 128ull * kb;
                    tc_mma_bf16(tmem_base, a_lo, b_hi, idesc, 1u);
                }
            }
            tc_commit(bar);
        }
        TC_PROF(5);
        // the coordinates of the next pass's neighbors travel while the MMAs run
        float pt_next[3];
        load_point(n0_next, pt_next);
        if (cnt > 0) {
            // one thread polls for the MMAs (they have read the tiles, which the next pass overwrites); the others
            // wait at the block barrier, which costs no issue slots
            const bool ok = (tid != 0) || mbar_wait(bar, parity, poll_limit);
            parity ^= 1u;
            if (__syncthreads_or(ok ? 0 : 1)) failed = true;
        }
        TC_PROF(6);
        if (last_of_block) {
            epi = true;
            epi_nonempty = cur.hi > cur.lo;
            epi_m = cur.m;
            epi_cb = cb;
        }
        cur = nxt;
        cb = nxt_cb;
        t0 = nxt_t0;
        cur_valid = nxt_valid;
        n0 = n0_next;
#pragma unroll
        for (int x = 0; x < 3; ++x) pt[x] = pt_next[x];
    }
#ifdef PCCNN_TC_PROFILE
    if (blockIdx.x == 0 && tid == 0)
        for (int i = 0; i < 8; ++i) g_tc_prof[i] = prof_[i];
#endif
    if (failed && tid == 0) {
        atomicExch(status, 5);
        mbar_wait(bar, parity ^ 1u, poll_limit);  // once more, bounded: MMAs still in flight must not outlive tensor memory
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

template <int NB>
struct TcBackwardSmem {
    static constexpr int kF = 2 * kTcRows * 128;  // F plane: 32 KB
    static constexpr int kBT = 2 * NB * 128;      // BT plane: two 64-neighbor blocks of [NB x 128 B]
    static constexpr int kGP = 2 * NB * 128;      // GP plane: two 64-channel blocks of [NB x 128 B]
    static constexpr int kFHi = 0, kFLo = kF, kBTHi = 2 * kF, kBTLo = kBTHi + kBT, kGPHi = kBTLo + kBT, kGPLo = kGPHi + kGP;
    static constexpr int kTiles = kGPLo + kGP;
    static constexpr int kMisc = 4096;  // barrier, tensor-memory slot, neighbor ids, basis parameters, parameter gradients
    static constexpr int kBytes = kTiles + kMisc;
};

// Everything of the backward pass that runs per neighbor pair, given dP = g W^T (rows of `inner` floats) for the
// samples [m_begin, m_end): dF (reduced into d_feat), db -> basis / offset / point / parameter gradients, and, when
// p_hi is given (Cin <= 128), the projected features P of the samples for the weight-gradient contraction, which
// share the gathered tile.  Three products per pass, all from the tiles F, BT (basis, [k][neighbor]) and GP (the
// sample's dP row, [k][channel]):
//     P^T [channel, k]          = F^T  * BT^T     A = F  MN-major, B = BT K-major      (accumulated over the passes)
//     db  [neighbor, k]         = F    * GP^T     A = F  K-major,  B = GP K-major      (accumulated over channel blocks)
//     dF^T[channel, neighbor]   = GP^T * BT       A = GP MN-major, B = BT MN-major     (one 16-deep step per 16 basis functions)
// A pass of this kernel is a chain of dependent phases, and with the few warps that fit an SM beside the tiles its
// duration is the number of instructions one warp has to run.  So the CTA has two groups of four warps that split
// every phase: threads 0-127 own one neighbor each (offset, basis, BT column, later the db row with the basis,
// offset, point and parameter gradients), threads 128-255 one channel each (GP column, most of the dF^T reduction,
// the P row); all eight warps copy feature rows.  The ids, coordinates and dP entries of the next pass are loaded
// while the products of this one run.
template <int NB, class BASIS, class ARGS>
__global__ void __launch_bounds__(256, 2)
backward_tc_kernel(ARGS args, int K, const float* __restrict__ pts, FeaturePlanes feats, int cin,
                   const float* __restrict__ samples, const int2* __restrict__ neighbors,
                   const int32_t* __restrict__ start_ids, const float* __restrict__ radii, int m_begin, int m_end,
                   const float* __restrict__ d_proj, float* __restrict__ d_feat, float* __restrict__ d_pts,
                   float* __restrict__ d_samples, float* __restrict__ d_param0, float* __restrict__ d_param1,
                   float* __restrict__ d_pdf, __nv_bfloat16* __restrict__ p_hi, __nv_bfloat16* __restrict__ p_lo, int ld_p,
                   uint32_t poll_limit, int* __restrict__ status) {
    using SM = TcBackwardSmem<NB>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];  // the swizzled tiles need 1024-byte alignment
    uint8_t* smem = smem_raw;
    uint8_t* misc = smem + SM::kTiles;
    uint64_t* bar = (uint64_t*)misc;
    uint32_t* tmem_slot = (uint32_t*)(misc + 8);
    int* s_n0 = (int*)(misc + 64);                      // [2][128]: the ids of this pass and of the next one
    float* s_params = (float*)(misc + 64 + 1024);       // up to 256 floats
    float* s_grad = (float*)(misc + 64 + 1024 + 1024);  // up to 256 floats
    static_assert(BASIS::kParamFloats <= 256 && BASIS::kGradFloats <= 256, "basis parameters do not fit their slots");
    static_assert(64 + 3 * 1024 <= SM::kMisc, "the small buffers do not fit");
    constexpr uint32_t kTmemCols = 256;  // db in columns [0, NB), P^T in [64, 64 + NB), dF^T in [128, 256)
    constexpr uint32_t kColP = 64, kColF = 128;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int grp = tid >> 7;   // 0: one neighbor per thread, 1: one channel per thread
    const int r = tid & 127;    // that neighbor / channel; also this thread's tensor-memory lane
    const int quad = warp & 3;  // the 32 tensor-memory lanes this warp may read
    if (tid == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    BASIS::load_params(s_params, args, K);
    for (int i = tid; i < BASIS::kGradFloats; i += 256) s_grad[i] = 0.f;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_lanes = tmem_base + ((uint32_t)(quad * 32) << 16);

    float inv[3];
#pragma unroll
    for (int d = 0; d < 3; ++d) inv[d] = BASIS::kUsesOffset ? __frcp_rn(__ldg(radii + d)) : 0.f;
    const int inner = cin * K;
    const bool with_p = p_hi != nullptr;
    const uint32_t f_hi = smem_u32(smem + SM::kFHi), f_lo = smem_u32(smem + SM::kFLo);
    const uint32_t bt_hi = smem_u32(smem + SM::kBTHi), bt_lo = smem_u32(smem + SM::kBTLo);
    const uint32_t gp_hi = smem_u32(smem + SM::kGPHi), gp_lo = smem_u32(smem + SM::kGPLo);
    constexpr uint32_t kBase = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 4) << 24);  // fp32 += bf16 x bf16, M = 128
    constexpr uint32_t idesc_p = kBase | (1u << 15) | ((uint32_t)(NB >> 3) << 17);                  // A MN-major, N = NB
    constexpr uint32_t idesc_db = kBase | ((uint32_t)(NB >> 3) << 17);                              // K-major, N = NB
    constexpr uint32_t idesc_df = kBase | (1u << 15) | (1u << 16) | ((uint32_t)(128 >> 3) << 17);   // both MN-major, N = 128
    uint32_t parity = 0;
    bool failed = false;
    // Parameter gradients: with a small basis every neighbor thread keeps its own partial sums in registers and the
    // block reduces them once at the end; a chain of warp reductions per pass would dominate a kernel that has
    // few warps to hide it.  Larger bases reduce per pass in shared memory.
    constexpr bool kLocalGrads = NB <= 16;
    float g_acc[kLocalGrads ? BASIS::kGradFloats : 1];
#pragma unroll
    for (int i = 0; i < (kLocalGrads ? BASIS::kGradFloats : 1); ++i) g_acc[i] = 0.f;
    // the dP entries of the next pass travel in registers while a small basis leaves room for them
    constexpr bool kPrefetchGP = NB <= 32;

    struct Sample {
        int m, lo, hi;
        float s[3];
    };
    auto load_sample = [&](int m) {
        Sample q;
        q.m = m;
        q.lo = q.hi = 0;
        q.s[0] = q.s[1] = q.s[2] = 0.f;
        if (m < m_end) {
            q.lo = (m > 0) ? __ldg(start_ids + m - 1) : 0;
            q.hi = __ldg(start_ids + m);
#pragma unroll
            for (int d = 0; d < 3; ++d) q.s[d] = BASIS::kUsesOffset ? __ldg(samples + (int64_t)m * 3 + d) : 0.f;
        }
        return q;
    };
    // `cur` becomes the next sample that has neighbors; a sample without any gets its row of zeros in P here
    Sample cur = load_sample(m_begin + blockIdx.x);
    Sample ahead = load_sample(cur.m + gridDim.x);
    auto open_sample = [&]() {
        while (cur.m < m_end && cur.hi == cur.lo) {
            if (with_p && grp == 1) {
                const size_t prow = (size_t)(cur.m - m_begin) * ld_p;
                for (int c = r; c < ld_p; c += 128) {
                    p_hi[prow + c] = __float2bfloat16_rn(0.f);
                    p_lo[prow + c] = __float2bfloat16_rn(0.f);
                }
            }
            cur = ahead;
            ahead = load_sample(cur.m + gridDim.x);
        }
    };
    auto load_id = [&](const Sample& q, int t0) { return (q.m < m_end && t0 + r < q.hi) ? __ldg(&neighbors[t0 + r]).x : -1; };
    auto load_point = [&](int n0, float (&q)[3]) {
#pragma unroll
        for (int x = 0; x < 3; ++x) q[x] = (BASIS::kUsesOffset && n0 >= 0) ? __ldg(pts + (int64_t)n0 * 3 + x) : 0.f;
    };
    // dP entries [k] of channel c of a sample
    auto load_gp = [&](const Sample& q, int c, float (&g)[NB]) {
        const float* grow = d_proj + (size_t)(q.m - m_begin) * inner;
        if (q.m < m_end && c < cin) {
            if (K == NB) {
#pragma unroll
                for (int k = 0; k < NB; k += 4) {
                    const float4 v = __ldg(reinterpret_cast<const float4*>(grow + (size_t)c * K + k));
                    g[k] = v.x; g[k + 1] = v.y; g[k + 2] = v.z; g[k + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int k = 0; k < NB; ++k) g[k] = (k < K) ? __ldg(grow + (size_t)c * K + k) : 0.f;
            }
        } else {
#pragma unroll
            for (int k = 0; k < NB; ++k) g[k] = 0.f;
        }
    };

    open_sample();
    int t0 = cur.lo, cb = 0, buf = 0;
    int n0 = -1;
    float pt[3] = {0.f, 0.f, 0.f}, d[3] = {0.f, 0.f, 0.f}, ds_acc[3] = {0.f, 0.f, 0.f};
    float gp[kPrefetchGP ? NB : 1];
    if (grp == 0) {
        n0 = load_id(cur, t0);
        s_n0[r] = n0;
        load_point(n0, pt);
    } else if constexpr (kPrefetchGP) {
        load_gp(cur, r, gp);
    }
    __syncthreads();

    while (cur.m < m_end && !failed) {
        const int cnt = min(kTcRows, cur.hi - t0);
        const int rows = (cnt + 15) & ~15;
        const int* ids = s_n0 + buf * kTcRows;
        const int t = t0 + r;
        const bool active = grp == 0 && r < cnt;
        const bool last_cb = cb + kTcChan >= cin;
        const bool last_pass = last_cb && t0 + kTcRows >= cur.hi;

        // ---- the pass after this one
        Sample nxt = cur;
        int nxt_t0 = t0, nxt_cb = cb + kTcChan;
        if (last_cb) {
            nxt_cb = 0;
            nxt_t0 = t0 + kTcRows;
        }
        gather_features_async<true, 8>(f_hi, f_lo, ids, rows, feats, cb);
        if (last_pass) {
            const Sample done = cur;
            cur = ahead;
            ahead = load_sample(cur.m + gridDim.x);
            open_sample();
            nxt = cur;
            nxt_t0 = nxt.lo;
            cur = done;
        }
        int n0_next = n0;
        if (grp == 0 && last_cb) n0_next = load_id(nxt, nxt_t0);

        if (grp == 0) {
            if (cb == 0) {
                // ---- offset, basis, BT column of this thread's pair, while the copies are in flight
                float b[NB];
                if (active) {
#pragma unroll
                    for (int x = 0; x < 3; ++x) d[x] = BASIS::kUsesOffset ? (pt[x] - cur.s[x]) * inv[x] : 0.f;
                    BASIS::eval(s_params, args, K, d, n0, t, cur.m, b);
                } else {
#pragma unroll
                    for (int k = 0; k < NB; ++k) b[k] = 0.f;
                }
                // all 128 columns are written: dF^T is computed for every column of the tile
                uint8_t* base_hi = smem + SM::kBTHi + (r >> 6) * (NB * 128) + (r & 7) * 2;
                uint8_t* base_lo = smem + SM::kBTLo + (r >> 6) * (NB * 128) + (r & 7) * 2;
                const int chunk = (r & 63) >> 3;
#pragma unroll
                for (int k = 0; k < NB; ++k) {
                    const __nv_bfloat16 h = __float2bfloat16_rn(b[k]);
                    const uint32_t off = sw128_offset(k, chunk);
                    *reinterpret_cast<__nv_bfloat16*>(base_hi + off) = h;
                    *reinterpret_cast<__nv_bfloat16*>(base_lo + off) = __float2bfloat16_rn(b[k] - __bfloat162float(h));
                }
            }
        } else {
            // ---- the dP entries of channel cb + r -> GP column r
            float g[NB];
            if constexpr (kPrefetchGP) {
#pragma unroll
                for (int k = 0; k < NB; ++k) g[k] = gp[k];
            } else {
                load_gp(cur, cb + r, g);
            }
            uint8_t* base_hi = smem + SM::kGPHi + (r >> 6) * (NB * 128) + (r & 7) * 2;
            uint8_t* base_lo = smem + SM::kGPLo + (r >> 6) * (NB * 128) + (r & 7) * 2;
            const int chunk = (r & 63) >> 3;
#pragma unroll
            for (int k = 0; k < NB; ++k) {
                const __nv_bfloat16 h = __float2bfloat16_rn(g[k]);
                const uint32_t off = sw128_offset(k, chunk);
                *reinterpret_cast<__nv_bfloat16*>(base_hi + off) = h;
                *reinterpret_cast<__nv_bfloat16*>(base_lo + off) = __float2bfloat16_rn(g[k] - __bfloat162float(h));
            }
        }
        cp_async_wait_all();
        fence_smem_to_async_proxy();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            // db[neighbor, k] (+)= F[neighbor, c] * dP[c, k]: 8 steps of 16 channels, accumulated over the blocks
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint64_t a_off = (uint64_t)(ks >> 2) * ((kTcRows * 128) >> 4) + 2ull * (ks & 3);
                const uint64_t b_off = (uint64_t)(ks >> 2) * ((NB * 128) >> 4) + 2ull * (ks & 3);
                const uint64_t a_hi = umma_desc_k_sw128(f_hi) + a_off, a_lo = umma_desc_k_sw128(f_lo) + a_off;
                const uint64_t b_hi = umma_desc_k_sw128(gp_hi) + b_off, b_lo = umma_desc_k_sw128(gp_lo) + b_off;
                tc_mma_bf16(tmem_base, a_hi, b_hi, idesc_db, (cb > 0 || ks > 0) ? 1u : 0u);
                tc_mma_bf16(tmem_base, a_lo, b_hi, idesc_db, 1u);
                tc_mma_bf16(tmem_base, a_hi, b_lo, idesc_db, 1u);
            }
            // dF^T[c, neighbor] = dP[c, k] * b[neighbor, k]: both operands MN-major (16 basis rows = 2048 bytes
            // = +128 per step; 64-channel / 64-neighbor groups are one block of NB rows apart)
#pragma unroll
            for (int ks = 0; ks < NB / 16; ++ks) {
                const uint64_t a_hi = umma_desc_mn_sw128(gp_hi, NB * 128) + 128ull * ks;
                const uint64_t a_lo = umma_desc_mn_sw128(gp_lo, NB * 128) + 128ull * ks;
                const uint64_t b_hi = umma_desc_mn_sw128(bt_hi, NB * 128) + 128ull * ks;
                const uint64_t b_lo = umma_desc_mn_sw128(bt_lo, NB * 128) + 128ull * ks;
                tc_mma_bf16(tmem_base + kColF, a_hi, b_hi, idesc_df, ks > 0 ? 1u : 0u);
                tc_mma_bf16(tmem_base + kColF, a_lo, b_hi, idesc_df, 1u);
                tc_mma_bf16(tmem_base + kColF, a_hi, b_lo, idesc_df, 1u);
            }
            if (with_p) {
                // P^T[c, k] (+)= F[neighbor, c] * b[neighbor, k] over the neighbors of this pass
                const bool first = t0 == cur.lo;
                // not unrolled: with this kernel's register budget the compiler's four-fold unrolled body issued
                // products with wrong operands (caught by the parity tests on samples of 49 - 64 neighbors)
#pragma unroll 1
                for (int kb = 0; kb < rows / 16; ++kb) {
                    const uint64_t a_hi = umma_desc_mn_sw128(f_hi, kTcRows * 128) + 128ull * kb;
                    const uint64_t a_lo = umma_desc_mn_sw128(f_lo, kTcRows * 128) + 128ull * kb;
                    const uint64_t b_off = (uint64_t)(kb >> 2) * ((NB * 128) >> 4) + 2ull * (kb & 3);
                    const uint64_t b_hi = umma_desc_k_sw128(bt_hi) + b_off, b_lo = umma_desc_k_sw128(bt_lo) + b_off;
                    tc_mma_bf16(tmem_base + kColP, a_hi, b_hi, idesc_p, (!first || kb > 0) ? 1u : 0u);
                    tc_mma_bf16(tmem_base + kColP, a_hi, b_lo, idesc_p, 1u);
                    tc_mma_bf16(tmem_base + kColP, a_lo, b_hi, idesc_p, 1u);
                }
            }
            tc_commit(bar);
        }
        // ---- loads of the next pass travel while the products run
        float pt_next[3] = {pt[0], pt[1], pt[2]};
        if (grp == 0) {
            if (last_cb) load_point(n0_next, pt_next);
        } else if constexpr (kPrefetchGP) {
            load_gp(nxt, nxt_cb + r, gp);
        }
        const bool ok = (tid != 0) || mbar_wait(bar, parity, poll_limit);
        parity ^= 1u;
        if (__syncthreads_or(ok ? 0 : 1)) {
            failed = true;
            break;
        }
        tc_fence_after();

        // ---- dF^T rows: a warp holds 32 consecutive channels as lanes, one column per neighbor, 32 columns at a
        // time; every reduction below is one 128-byte line of a neighbor's feature-gradient row
        auto reduce_df = [&](int j0) {
            if (j0 >= cnt) return;
            // the ids first: a reduction orders memory operations, so a shared-memory read per column inside the loop
            // below could not be moved ahead of the previous column's reduction
            int idr[32];
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
                const int4 q = *reinterpret_cast<const int4*>(ids + j0 + j);
                idr[j] = q.x; idr[j + 1] = q.y; idr[j + 2] = q.z; idr[j + 3] = q.w;
            }
            uint32_t v[32];
            tc_ld_32x32(tmem_lanes + kColF + (uint32_t)j0, v);
            const int c = cb + r;
            if (c < cin) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (j0 + j < cnt) atomicAdd(d_feat + (int64_t)idr[j] * cin + c, __uint_as_float(v[j]));
                }
            }
        };
        if (grp == 1) {
            reduce_df(0);
            reduce_df(32);
            reduce_df(64);
            if (last_pass && with_p) {
                // ---- P row of the sample: thread = channel, NB accumulator columns -> K entries
                float acc[NB];
#pragma unroll
                for (int k0 = 0; k0 < NB; k0 += 16) {
                    uint32_t v[16];
                    tc_ld_32x16(tmem_lanes + kColP + (uint32_t)k0, v);
#pragma unroll
                    for (int k = 0; k < 16; ++k) acc[k0 + k] = __uint_as_float(v[k]);
                }
                const size_t prow = (size_t)(cur.m - m_begin) * ld_p;
                store_p_row<NB>(acc, r, cin, K, p_hi, p_lo, prow);
                for (int c = inner + r; c < ld_p; c += 128) {
                    p_hi[prow + c] = __float2bfloat16_rn(0.f);
                    p_lo[prow + c] = __float2bfloat16_rn(0.f);
                }
            }
        } else {
            if (last_cb) {
                // ---- db row of this thread's pair -> basis gradient, offset gradient, point gradients
                float db[NB];
#pragma unroll
                for (int k0 = 0; k0 < NB; k0 += 16) {
                    uint32_t v[16];
                    tc_ld_32x16(tmem_lanes + (uint32_t)k0, v);
#pragma unroll
                    for (int k = 0; k < 16; ++k) db[k0 + k] = active ? __uint_as_float(v[k]) : 0.f;
                }
                float d_off[3] = {0.f, 0.f, 0.f}, dpdf = 0.f;
                if constexpr (kLocalGrads)
                    BASIS::grad_local(s_params, args, K, d, max(n0, 0), t, cur.m, active, db, d_off, g_acc, dpdf);
                else
                    BASIS::grad(s_params, args, K, d, max(n0, 0), t, cur.m, active, db, d_off, s_grad, dpdf);
                if (active) {
#pragma unroll
                    for (int x = 0; x < 3; ++x) {
                        const float gx = d_off[x] * inv[x];
                        if (d_pts && gx != 0.f) atomicAdd(d_pts + (int64_t)n0 * 3 + x, gx);
                        ds_acc[x] += gx;
                    }
                    if (d_pdf && dpdf != 0.f) atomicAdd(d_pdf + n0, dpdf);
                }
            }
            reduce_df(96);
            if (last_pass) {
                if (d_samples) {
#pragma unroll
                    for (int x = 0; x < 3; ++x) {
                        const float tot = warp_sum(ds_acc[x]);
                        if (lane == 0 && tot != 0.f) atomicAdd(d_samples + (int64_t)cur.m * 3 + x, -tot);
                    }
                }
                ds_acc[0] = ds_acc[1] = ds_acc[2] = 0.f;
            }
            s_n0[(buf ^ 1) * kTcRows + r] = n0_next;
        }
        tc_fence_before();
        __syncthreads();  // tiles, accumulators and the other id buffer are free; the next ids are staged
        if (last_cb) buf ^= 1;
        cur = nxt;
        t0 = nxt_t0;
        cb = nxt_cb;
        n0 = n0_next;
#pragma unroll
        for (int x = 0; x < 3; ++x) pt[x] = pt_next[x];
    }
    if (failed && tid == 0) {
        atomicExch(status, 6);
        mbar_wait(bar, parity ^ 1u, poll_limit);
    }
    if constexpr (kLocalGrads) {
        if (grp == 0) {
#pragma unroll
            for (int i = 0; i < BASIS::kGradFloats; ++i) {
                const float tot = warp_sum(g_acc[i]);
                if (lane == 0 && tot != 0.f) atomicAdd(s_grad + i, tot);
            }
        }
    }
    __syncthreads();
    BASIS::flush(s_grad, K, d_param0, d_param1);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---- host side ------------------------------------------------------------------------------
// Poll limit of the bounded waits (gemm.cu owns it, together with the test hook that shortens it).
uint32_t tensor_core_poll_limit();

template <int NB, class BASIS, class ARGS, bool SPLIT_F, bool HALF = false>
static int launch_project_tc_nb(int K, const ARGS& args, const float* pts, const FeaturePlanes& feats, int cin, const float* samples,
                                const int32_t* neighbors, const int32_t* start_ids, const float* radii, int m_begin,
                                int m_end, void* p_hi, void* p_lo, int ld_p, int* status, cudaStream_t s) {
    if (!HALF && cin <= 64)  // one 64-channel block per plane: a smaller CTA, more of them per SM
        return launch_project_tc_nb<NB, BASIS, ARGS, SPLIT_F, true>(K, args, pts, feats, cin, samples, neighbors, start_ids,
                                                                    radii, m_begin, m_end, p_hi, p_lo, ld_p, status, s);
    using SM = TcForwardSmem<NB, SPLIT_F, HALF>;
    auto kernel = project_tc_kernel<NB, BASIS, ARGS, SPLIT_F, HALF>;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [&] {
        attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kBytes);
    });
    PCCNN_CUDA(attr_err);
    const int per_sm = (227 * 1024) / (SM::kBytes + 1024);
    const int64_t cap = (int64_t)sm_count() * (per_sm < 1 ? 1 : per_sm);
    const int count = m_end - m_begin;
    const unsigned grid = (unsigned)(count < cap ? count : cap);
    kernel<<<grid, 128, SM::kBytes, s>>>(args, K, pts, feats, cin, samples, (const int2*)neighbors, start_ids,
                                                        radii, m_begin, m_end, (__nv_bfloat16*)p_hi, (__nv_bfloat16*)p_lo,
                                                        ld_p, tensor_core_poll_limit(), status);
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

// Tensor-core projection of the samples [m_begin, m_end) (3-D points, K <= 64).
template <class ARGS, template <int, int> class BASIS, bool SPLIT_F>
static int launch_project_tc(int K, const ARGS& args, const float* pts, const FeaturePlanes& feats, int cin, const float* samples,
                             const int32_t* neighbors, const int32_t* start_ids, const float* radii, int m_begin,
                             int m_end, void* p_hi, void* p_lo, int ld_p, int* status, cudaStream_t s) {
    if (m_end <= m_begin) return PCCNN_OK;
    if (K <= 16)
        return launch_project_tc_nb<16, BASIS<3, 16>, ARGS, SPLIT_F>(K, args, pts, feats, cin, samples, neighbors, start_ids,
                                                                         radii, m_begin, m_end, p_hi, p_lo, ld_p, status, s);
    if (K <= 32)
        return launch_project_tc_nb<32, BASIS<3, 32>, ARGS, SPLIT_F>(K, args, pts, feats, cin, samples, neighbors, start_ids,
                                                                         radii, m_begin, m_end, p_hi, p_lo, ld_p, status, s);
    return launch_project_tc_nb<64, BASIS<3, 64>, ARGS, SPLIT_F>(K, args, pts, feats, cin, samples, neighbors, start_ids,
                                                                     radii, m_begin, m_end, p_hi, p_lo, ld_p, status, s);
}

template <int NB, class BASIS, class ARGS>
static int launch_backward_tc_nb(int K, const ARGS& args, const float* pts, const FeaturePlanes& feats, int cin,
                                 const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                                 const float* radii, int m_begin, int m_end, const float* d_proj, float* d_feat,
                                 float* d_pts, float* d_samples, float* d_param0, float* d_param1, float* d_pdf,
                                 void* p_hi, void* p_lo, int ld_p, int* status, cudaStream_t s) {
    auto kernel = backward_tc_kernel<NB, BASIS, ARGS>;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [&] {
        attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TcBackwardSmem<NB>::kBytes);
    });
    PCCNN_CUDA(attr_err);
    const int count = m_end - m_begin;
    // two CTAs per SM: 2 x 256 tensor-memory columns and 2 x (tiles + 1 KB) of shared memory
    const int per_sm = (227 * 1024) / (TcBackwardSmem<NB>::kBytes + 1024) >= 2 ? 2 : 1;
    const int64_t cap = (int64_t)sm_count() * per_sm;
    const unsigned grid = (unsigned)(count < cap ? count : cap);
    kernel<<<grid, 256, TcBackwardSmem<NB>::kBytes, s>>>(args, K, pts, feats, cin, samples, (const int2*)neighbors, start_ids,
                                                         radii, m_begin, m_end, d_proj, d_feat, d_pts, d_samples, d_param0,
                                                         d_param1, d_pdf, (__nv_bfloat16*)p_hi, (__nv_bfloat16*)p_lo, ld_p,
                                                         tensor_core_poll_limit(), status);
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

template <class ARGS, template <int, int> class BASIS>
static int launch_backward_tc(int K, const ARGS& args, const float* pts, const FeaturePlanes& feats, int cin, const float* samples,
                              const int32_t* neighbors, const int32_t* start_ids, const float* radii, int m_begin,
                              int m_end, const float* d_proj, float* d_feat, float* d_pts, float* d_samples,
                              float* d_param0, float* d_param1, float* d_pdf, void* p_hi, void* p_lo, int ld_p, int* status,
                              cudaStream_t s) {
    if (m_end <= m_begin) return PCCNN_OK;
    if (K <= 16)
        return launch_backward_tc_nb<16, BASIS<3, 16>, ARGS>(K, args, pts, feats, cin, samples, neighbors, start_ids, radii,
                                                             m_begin, m_end, d_proj, d_feat, d_pts, d_samples, d_param0,
                                                             d_param1, d_pdf, p_hi, p_lo, ld_p, status, s);
    if (K <= 32)
        return launch_backward_tc_nb<32, BASIS<3, 32>, ARGS>(K, args, pts, feats, cin, samples, neighbors, start_ids, radii,
                                                             m_begin, m_end, d_proj, d_feat, d_pts, d_samples, d_param0,
                                                             d_param1, d_pdf, p_hi, p_lo, ld_p, status, s);
    return launch_backward_tc_nb<64, BASIS<3, 64>, ARGS>(K, args, pts, feats, cin, samples, neighbors, start_ids, radii,
                                                         m_begin, m_end, d_proj, d_feat, d_pts, d_samples, d_param0,
                                                         d_param1, d_pdf, p_hi, p_lo, ld_p, status, s);
}

// ---- projection without a neighbor list -----------------------------------------------------------------------
// The same P rows as project_tc_kernel, for callers that hold the grid instead of a neighbor list: the CTA finds the
// neighbors of its sample itself -- the candidate ranges of the sample's 27-cell stencil (find_ranges_grid_ds.cu:
// 65-166 of the reference, resolved as the search kernel does), the radius predicate of count_neighbors.cu:87 with its
// exact operation order -- compacts the hits in ascending position and runs the tensor-core pass on every 128 of
// them.  The list [T, 2] is never written or read.  Points and feature planes are in grid order (sorted position =
// row), samples in any order.
template <int NB, class BASIS, class ARGS, bool SPLIT_F>
__global__ void __launch_bounds__(128)
project_tc_grid_kernel(ARGS args, int K, int num_pts, const float* __restrict__ sorted_pts,
                       const int64_t* __restrict__ sorted_keys, FeaturePlanes feats, int cin, int num_samples,
                       const float* __restrict__ samples, const int64_t* __restrict__ sample_keys,
                       const int2* __restrict__ grid_ds, const int32_t* __restrict__ grid_size,
                       const float* __restrict__ radii, int m_begin, int m_end, __nv_bfloat16* __restrict__ p_hi,
                       __nv_bfloat16* __restrict__ p_lo, int ld_p, uint32_t poll_limit, int* __restrict__ status) {
    using SM = TcForwardSmem<NB, SPLIT_F>;
    using S = Stencil<3>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    uint8_t* misc = smem + SM::kTiles;
    uint64_t* bar = (uint64_t*)misc;
    uint32_t* tmem_slot = (uint32_t*)(misc + 8);
    int* s_warp_hits = (int*)(misc + 16);          // [4]
    int* s_lo = (int*)(misc + 32);                 // [9]
    int* s_pref = (int*)(misc + 32 + 40);          // [10]
    int* s_n0 = (int*)(misc + 128);                // [128] ids of the pass being run
    float* s_params = (float*)(misc + 128 + 512);  // up to 256 floats
    int* s_q_id = (int*)(misc + 128 + 512 + 1024); // [256] hits waiting for a pass: up to 127 left over + 128 new ones
    static_assert(BASIS::kParamFloats <= 256, "basis parameters do not fit the shared-memory slot");
    constexpr uint32_t kTmemCols = NB < 32 ? 32 : NB;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    BASIS::load_params(s_params, args, K);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const GridDesc<3> g = load_grid<3>(grid_size);
    float inv[3];
#pragma unroll
    for (int d = 0; d < 3; ++d) inv[d] = __frcp_rn(__ldg(radii + d));
    const int inner = cin * K;
    const uint32_t f_hi = smem_u32(smem + SM::kFHi), f_lo = smem_u32(smem + SM::kFLo);
    const uint32_t bt_hi = smem_u32(smem + SM::kBTHi), bt_lo = smem_u32(smem + SM::kBTLo);
    constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(NB >> 3) << 17) |
                               ((uint32_t)(128 >> 4) << 24);
    uint32_t parity = 0;
    bool failed = false;

    for (int m = m_begin + blockIdx.x; m < m_end && !failed; m += gridDim.x) {
        float s[3];
#pragma unroll
        for (int d = 0; d < 3; ++d) s[d] = __ldg(samples + (int64_t)m * 3 + d);
        const size_t row = (size_t)(m - m_begin) * ld_p;
        int num_cand = 0;
        if (warp == 0) num_cand = resolve_ranges<3>(__ldg(sample_keys + m), g, grid_ds, sorted_keys, num_pts, s_lo, s_pref);
        __syncthreads();
        num_cand = s_pref[S::kRanges];

        for (int cb = 0; cb < cin && !failed; cb += kTcChan) {
            bool first = true;
            int queued = 0;  // hits waiting in s_q_id
            int base = 0;    // candidates tested so far
            while (true) {
                // ---- 128 candidates: exact radius test, hits appended to the queue in ascending position
                if (base < num_cand) {
                    const int gidx = base + tid;
                    bool hit = false;
                    int j = 0;
                    if (gidx < num_cand) {
                        int r = 0;
                        while (gidx >= s_pref[r + 1]) ++r;
                        j = s_lo[r] + gidx - s_pref[r];
                        float acc = 0.f;
#pragma unroll
                        for (int d = 0; d < 3; ++d) {
                            const float v = __fmul_rn(__fsub_rn(s[d], __ldg(sorted_pts + (int64_t)j * 3 + d)), inv[d]);
                            acc = (d == 0) ? __fmul_rn(v, v) : __fmaf_rn(v, v, acc);
                        }
                        hit = acc < 1.0f;
                    }
                    const unsigned bal = __ballot_sync(kFullMask, hit);
                    if (lane == 0) s_warp_hits[warp] = __popc(bal);
                    __syncthreads();
                    int before = queued;
                    for (int w = 0; w < warp; ++w) before += s_warp_hits[w];
                    if (hit) s_q_id[before + __popc(bal & ((1u << lane) - 1u))] = j;
                    queued += s_warp_hits[0] + s_warp_hits[1] + s_warp_hits[2] + s_warp_hits[3];
                    base += 128;
                    __syncthreads();
                }
                const bool all_tested = base >= num_cand;
                if (queued < kTcRows && !all_tested) continue;
                if (queued == 0) break;

                // ---- one pass over the first min(128, queued) hits
                const int cnt = min(kTcRows, queued);
                const int rows = (cnt + 15) & ~15;
                const int n0 = tid < cnt ? s_q_id[tid] : -1;
                const int moved = tid + kTcRows < queued ? s_q_id[tid + kTcRows] : -1;  // does not fit this pass
                s_n0[tid] = n0;
                __syncthreads();
                if (moved >= 0) s_q_id[tid] = moved;  // the queue's tail moves to its front
                queued -= cnt;
                gather_features_async<SPLIT_F>(f_hi, f_lo, s_n0, rows, feats, cb);
                {
                    float b[NB];
                    if (tid < cnt) {
                        float d[3];
#pragma unroll
                        for (int x = 0; x < 3; ++x) d[x] = (__ldg(sorted_pts + (int64_t)n0 * 3 + x) - s[x]) * inv[x];
                        BASIS::eval(s_params, args, K, d, n0, 0, m, b);
                    } else {
#pragma unroll
                        for (int k = 0; k < NB; ++k) b[k] = 0.f;
                    }
                    if (tid < rows) {
                        uint8_t* base_hi = smem + SM::kBTHi + (tid >> 6) * (NB * 128) + (tid & 7) * 2;
                        uint8_t* base_lo = smem + SM::kBTLo + (tid >> 6) * (NB * 128) + (tid & 7) * 2;
                        const int chunk = (tid & 63) >> 3;
#pragma unroll
                        for (int k = 0; k < NB; ++k) {
                            const __nv_bfloat16 h = __float2bfloat16_rn(b[k]);
                            const uint32_t off = sw128_offset(k, chunk);
                            *reinterpret_cast<__nv_bfloat16*>(base_hi + off) = h;
                            *reinterpret_cast<__nv_bfloat16*>(base_lo + off) = __float2bfloat16_rn(b[k] - __bfloat162float(h));
                        }
                    }
                }
                cp_async_wait_all();
                fence_smem_to_async_proxy();
                __syncthreads();
                if (tid == 0) {
                    tc_fence_after();
                    for (int kb = 0; kb < rows / 16; ++kb) {
                        const uint64_t a_hi = umma_desc_mn_sw128(f_hi, kTcRows * 128) + 128ull * kb;
                        const uint64_t b_off = (uint64_t)(kb >> 2) * ((NB * 128) >> 4) + 2ull * (kb & 3);
                        const uint64_t b_hi = umma_desc_k_sw128(bt_hi) + b_off, b_lo = umma_desc_k_sw128(bt_lo) + b_off;
                        tc_mma_bf16(tmem_base, a_hi, b_hi, idesc, (!first || kb > 0) ? 1u : 0u);
                        tc_mma_bf16(tmem_base, a_hi, b_lo, idesc, 1u);
                        if (SPLIT_F) {
                            const uint64_t a_lo = umma_desc_mn_sw128(f_lo, kTcRows * 128) + 128ull * kb;
                            tc_mma_bf16(tmem_base, a_lo, b_hi, idesc, 1u);
                        }
                    }
                    tc_commit(bar);
                }
                const bool ok = (tid != 0) || mbar_wait(bar, parity, poll_limit);
                parity ^= 1u;
                if (__syncthreads_or(ok ? 0 : 1)) {
                    failed = true;
                    break;
                }
                first = false;
            }
            if (failed) break;
            // ---- epilogue: thread = channel cb + tid
            tc_fence_after();
            float acc[NB];
            if (first) {
#pragma unroll
                for (int k = 0; k < NB; ++k) acc[k] = 0.f;
            } else {
#pragma unroll
                for (int k0 = 0; k0 < NB; k0 += 16) {
                    uint32_t r[16];
                    tc_ld_32x16(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)k0, r);
#pragma unroll
                    for (int k = 0; k < 16; ++k) acc[k0 + k] = __uint_as_float(r[k]);
                }
            }
            store_p_row<NB>(acc, cb + tid, cin, K, p_hi, p_lo, row);
            tc_fence_before();
            __syncthreads();
        }
        for (int c = inner + tid; c < ld_p; c += 128) {
            p_hi[row + c] = __float2bfloat16_rn(0.f);
            if (p_lo) p_lo[row + c] = __float2bfloat16_rn(0.f);
        }
    }
    if (failed && tid == 0) {
        atomicExch(status, 7);
        mbar_wait(bar, parity ^ 1u, poll_limit);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// fp32 or bf16 rows src[map[r]] -> bf16 planes in row order r (hi, and lo for fp32 input): the feature planes in grid
// order for the list-free projection, where a neighbor is named by its sorted position.
template <class FT>
static __global__ void __launch_bounds__(256)
permute_features_kernel(int64_t rows, int cin, int ld, const FT* __restrict__ src, const int64_t* __restrict__ map,
                        __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo) {
    const int64_t total = rows * (ld / 8);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t r = i / (ld / 8);
        const int c = (int)(i - r * (ld / 8)) * 8;
        const int64_t from = map ? __ldg(map + r) : r;
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = (c + e < cin) ? (float)src[from * cin + c + e] : 0.f;
        uint32_t hw[4], lw[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
            const __nv_bfloat162 l2 = __floats2bfloat162_rn(v[2 * q] - __low2float(h2), v[2 * q + 1] - __high2float(h2));
            hw[q] = *reinterpret_cast<const uint32_t*>(&h2);
            lw[q] = *reinterpret_cast<const uint32_t*>(&l2);
        }
        *reinterpret_cast<uint4*>(hi + r * ld + c) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        if (lo) *reinterpret_cast<uint4*>(lo + r * ld + c) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
    }
}

template <int NB, class BASIS, class ARGS, bool SPLIT_F>
static int launch_project_tc_grid_nb(int K, const ARGS& args, int num_pts, const float* sorted_pts, const int64_t* sorted_keys,
                                     const FeaturePlanes& feats, int cin, int num_samples, const float* samples,
                                     const int64_t* sample_keys, const int32_t* grid_ds, const int32_t* grid_size,
                                     const float* radii, int m_begin, int m_end, void* p_hi, void* p_lo, int ld_p,
                                     int* status, cudaStream_t s) {
    auto kernel = project_tc_grid_kernel<NB, BASIS, ARGS, SPLIT_F>;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [&] {
        attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TcForwardSmem<NB, SPLIT_F>::kGridBytes);
    });
    PCCNN_CUDA(attr_err);
    const int per_sm = (227 * 1024) / (TcForwardSmem<NB, SPLIT_F>::kGridBytes + 1024);
    const int64_t cap = (int64_t)sm_count() * (per_sm < 1 ? 1 : per_sm);
    const int count = m_end - m_begin;
    const unsigned grid = (unsigned)(count < cap ? count : cap);
    kernel<<<grid, 128, TcForwardSmem<NB, SPLIT_F>::kGridBytes, s>>>(args, K, num_pts, sorted_pts, sorted_keys, feats, cin, num_samples, samples,
                                                        sample_keys, (const int2*)grid_ds, grid_size, radii, m_begin, m_end,
                                                        (__nv_bfloat16*)p_hi, (__nv_bfloat16*)p_lo, ld_p,
                                                        tensor_core_poll_limit(), status);
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

template <class ARGS, template <int, int> class BASIS, bool SPLIT_F>
static int launch_project_tc_grid(int K, const ARGS& args, int num_pts, const float* sorted_pts, const int64_t* sorted_keys,
                                  const FeaturePlanes& feats, int cin, int num_samples, const float* samples,
                                  const int64_t* sample_keys, const int32_t* grid_ds, const int32_t* grid_size,
                                  const float* radii, int m_begin, int m_end, void* p_hi, void* p_lo, int ld_p, int* status,
                                  cudaStream_t s) {
    if (m_end <= m_begin) return PCCNN_OK;
#define PCCNN_GRID_NB(NBV)                                                                                              \
    return launch_project_tc_grid_nb<NBV, BASIS<3, NBV>, ARGS, SPLIT_F>(K, args, num_pts, sorted_pts, sorted_keys, feats, cin, \
                                                                        num_samples, samples, sample_keys, grid_ds, grid_size, \
                                                                        radii, m_begin, m_end, p_hi, p_lo, ld_p, status, s)
    if (K <= 16) PCCNN_GRID_NB(16);
    if (K <= 32) PCCNN_GRID_NB(32);
    PCCNN_GRID_NB(64);
#undef PCCNN_GRID_NB
}

}  // namespace pccnn
