// Templates shared by the convolution operators (conv.cu: KPConv, MCConv; conv_variants_*.cu: the other basis
// functions of the reference): the projection kernels, the per-pair backward kernel, their launchers, and the
// forward / backward / weight-variance drivers, all parameterised by a basis functor.
#pragma once

#include <cuda_bf16.h>

#include <type_traits>

#include "common.cuh"
#include "gemm.cuh"
#include "status.cuh"
#include "conv_tc.cuh"

namespace pccnn {

// 0: the pair-level work runs on the tensor cores where those kernels apply (3-D points, at least 32 input
// channels); 1: CUDA-core kernels everywhere (kept for the other dimensions and narrow inputs, and selectable so
// that the two paths can be compared).  Defined in conv.cu, changed by pccnn_conv_set_path.
extern int g_conv_path;

static bool use_tensor_core_pairs(int D, int cin) { return g_conv_path == 0 && D == 3 && cin >= 32; }

// Warps per block: the two per-warp basis buffers of the backward kernel must fit in 48 KB.
template <int KP>
constexpr int conv_warps() { return KP >= 64 ? 2 : 4; }

struct KPBasisArgs {
    const float* kernel_pts;  // [K, D]
    float inv_sigma;
};
struct MLPBasisArgs {
    const float* axis;  // [D, H]
    const float* bias;  // [H]
    const float* pdf;   // [N]
};

// Basis functors: eval() fills b[0..K) for one pair given its normalised offset.
// Whether a basis may be instantiated for every point dimension or only for three.
template <template <int, int> class BASIS>
struct BasisTraits {
    static constexpr bool kOnly3D = false;
};

// Calls f(std::integral_constant<int, D>) for the run-time dimension D; bases that exist in 3-D only are
// not instantiated for the others.
template <bool ONLY3, class F>
static int dispatch_dims(int D, F&& f) {
    if constexpr (ONLY3) {
        if (D != 3) {
            set_error("this operator is defined for 3-D points only (got %d)", D);
            return PCCNN_ERR_INVALID;
        }
        return f(std::integral_constant<int, 3>{});
    } else {
        switch (D) {
            case 2: return f(std::integral_constant<int, 2>{});
            case 3: return f(std::integral_constant<int, 3>{});
            case 4: return f(std::integral_constant<int, 4>{});
            case 5: return f(std::integral_constant<int, 5>{});
            case 6: return f(std::integral_constant<int, 6>{});
            default:
                set_error("point dimension %d outside [2, 6]", D);
                return PCCNN_ERR_INVALID;
        }
    }
}

template <int D, int KP>
struct KPBasis {
    static constexpr bool kUsesOffset = true;  // eval / grad read the normalised offset d_t
    static constexpr int kParamFloats = KP * D;
    __device__ static void load_params(float* sp, const KPBasisArgs& a, int K) {
        for (int i = threadIdx.x; i < KP * D; i += blockDim.x) sp[i] = (i < K * D) ? __ldg(a.kernel_pts + i) : 0.f;
    }
    __device__ static void eval(const float* sp, const KPBasisArgs& a, int K, const float (&d)[D], int /*n0*/,
                                int /*t*/, int /*m*/, float (&b)[KP]) {
#pragma unroll
        for (int k = 0; k < KP; ++k) {
            float acc = 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) {
                const float v = sp[k * D + x] - d[x];
                acc = fmaf(v, v, acc);
            }
            const float val = 1.0f - sqrtf(fmaxf(acc, 0.f)) * a.inv_sigma;
            b[k] = (k < K) ? fminf(fmaxf(val, 0.f), 1.f) : 0.f;
        }
    }
    // Backward of eval (shared/kernel_pts_basis.cu:41-70 of the reference: mask 1 - dist/sigma >= 0,
    // 1 / (dist + 1e-6)).  db = dL/db[k]; adds to d_off = dL/d(offset) and, through shared-memory
    // float reductions, to s_grad laid out like the kernel points [K, D].
    static constexpr int kGradFloats = KP * D;
    // Called by all 32 lanes (inactive lanes pass active = false): the parameter gradients of the 32
    // pairs are summed with shuffles and lane 0 adds one value per entry to s_grad.
    __device__ static void grad(const float* sp, const KPBasisArgs& a, int K, const float (&d)[D], int /*n0*/,
                                int /*t*/, int /*m*/, bool active, const float* db, float (&d_off)[D], float* s_grad,
                                float& /*d_pdf*/) {
        const int lane = lane_id();
        for (int k = 0; k < K; ++k) {
            float v[D], acc = 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) {
                v[x] = sp[k * D + x] - d[x];
                acc = fmaf(v[x], v[x], acc);
            }
            const float dist = sqrtf(fmaxf(acc, 0.f));
            float gk = 0.f;
            if (active && 1.0f - dist * a.inv_sigma >= 0.f) gk = -db[k] * a.inv_sigma / (dist + 1e-6f);
            if (!__any_sync(kFullMask, gk != 0.f)) continue;
#pragma unroll
            for (int x = 0; x < D; ++x) {
                const float t = gk * v[x];
                d_off[x] -= t;
                const float tot = warp_sum(t);
                if (lane == 0) atomicAdd(s_grad + k * D + x, tot);
            }
        }
    }
    // Same gradient without any cross-lane work: the parameter gradients of this thread's pairs are added to its
    // own accumulators acc[kGradFloats] (laid out like s_grad), which the caller reduces once at the end.
    __device__ static void grad_local(const float* sp, const KPBasisArgs& a, int K, const float (&d)[D], int /*n0*/,
                                      int /*t*/, int /*m*/, bool active, const float* db, float (&d_off)[D],
                                      float (&acc_g)[kGradFloats], float& /*d_pdf*/) {
#pragma unroll
        for (int k = 0; k < KP; ++k) {
            float v[D], acc = 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) {
                v[x] = sp[k * D + x] - d[x];
                acc = fmaf(v[x], v[x], acc);
            }
            const float dist = sqrtf(fmaxf(acc, 0.f));
            float gk = 0.f;
            if (active && k < K && 1.0f - dist * a.inv_sigma >= 0.f) gk = -db[k] * a.inv_sigma / (dist + 1e-6f);
#pragma unroll
            for (int x = 0; x < D; ++x) {
                const float t = gk * v[x];
                d_off[x] -= t;
                acc_g[k * D + x] += t;
            }
        }
    }
    __device__ static void flush(const float* s_grad, int K, float* g0, float* /*g1*/) {
        for (int i = threadIdx.x; i < K * D; i += blockDim.x)
            if (s_grad[i] != 0.f) atomicAdd(g0 + i, s_grad[i]);
    }
};

template <int D, int KP>
struct MLPBasis {
    static constexpr bool kUsesOffset = true;
    static constexpr int kParamFloats = (D + 1) * KP;
    __device__ static void load_params(float* sp, const MLPBasisArgs& a, int K) {
        for (int i = threadIdx.x; i < (D + 1) * KP; i += blockDim.x) {
            const int row = i / KP, k = i - row * KP;
            float v = 0.f;
            if (k < K) v = (row < D) ? __ldg(a.axis + row * K + k) : __ldg(a.bias + k);
            sp[i] = v;
        }
    }
    __device__ static void eval(const float* sp, const MLPBasisArgs& a, int K, const float (&d)[D], int n0,
                                int /*t*/, int /*m*/, float (&b)[KP]) {
        const float inv_pdf = 1.0f / __ldg(a.pdf + n0);
#pragma unroll
        for (int k = 0; k < KP; ++k) {
            float acc = 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) acc = fmaf(d[x], sp[x * KP + k], acc);
            acc += sp[D * KP + k];
            acc = acc > 0.f ? acc : 0.2f * acc;
            b[k] = (k < K) ? acc * inv_pdf : 0.f;
        }
    }
    // Backward of eval (shared/mlp_basis.cu:50-96 of the reference).  s_grad holds the axis
    // gradient [D, KP] followed by the bias gradient [KP].
    static constexpr int kGradFloats = (D + 1) * KP;
    __device__ static void grad(const float* sp, const MLPBasisArgs& a, int K, const float (&d)[D], int n0,
                                int /*t*/, int /*m*/, bool active, const float* db, float (&d_off)[D], float* s_grad,
                                float& d_pdf) {
        const int lane = lane_id();
        const float inv_pdf = active ? 1.0f / __ldg(a.pdf + n0) : 0.f;
        for (int k = 0; k < K; ++k) {
            float pre = 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) pre = fmaf(d[x], sp[x * KP + k], pre);
            pre += sp[D * KP + k];
            const float act = pre > 0.f ? pre : 0.2f * pre;
            const float dbk = active ? db[k] : 0.f;
            d_pdf -= act * dbk * inv_pdf * inv_pdf;
            const float cur = dbk * inv_pdf * (act > 0.f ? 1.0f : 0.2f);
            if (!__any_sync(kFullMask, cur != 0.f)) continue;
            const float tot_b = warp_sum(cur);
            if (lane == 0) atomicAdd(s_grad + D * KP + k, tot_b);
#pragma unroll
            for (int x = 0; x < D; ++x) {
                d_off[x] = fmaf(cur, sp[x * KP + k], d_off[x]);
                const float tot = warp_sum(d[x] * cur);
                if (lane == 0) atomicAdd(s_grad + x * KP + k, tot);
            }
        }
    }
    __device__ static void grad_local(const float* sp, const MLPBasisArgs& a, int K, const float (&d)[D], int n0,
                                      int /*t*/, int /*m*/, bool active, const float* db, float (&d_off)[D],
                                      float (&acc_g)[kGradFloats], float& d_pdf) {
        const float inv_pdf = active ? 1.0f / __ldg(a.pdf + n0) : 0.f;
#pragma unroll
        for (int k = 0; k < KP; ++k) {
            float pre = 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) pre = fmaf(d[x], sp[x * KP + k], pre);
            pre += sp[D * KP + k];
            const float act = pre > 0.f ? pre : 0.2f * pre;
            const float dbk = (active && k < K) ? db[k] : 0.f;
            d_pdf -= act * dbk * inv_pdf * inv_pdf;
            const float cur = dbk * inv_pdf * (act > 0.f ? 1.0f : 0.2f);
            acc_g[D * KP + k] += cur;
#pragma unroll
            for (int x = 0; x < D; ++x) {
                d_off[x] = fmaf(cur, sp[x * KP + k], d_off[x]);
                acc_g[x * KP + k] = fmaf(d[x], cur, acc_g[x * KP + k]);
            }
        }
    }
    __device__ static void flush(const float* s_grad, int K, float* g_axis, float* g_bias) {
        for (int i = threadIdx.x; i < (D + 1) * KP; i += blockDim.x) {
            const int row = i / KP, k = i - row * KP;
            if (k < K && s_grad[i] != 0.f) atomicAdd(row < D ? g_axis + row * K + k : g_bias + k, s_grad[i]);
        }
    }
};

// P[m, c*K + k] for the samples [m_begin, m_end), written as bf16 hi (+ lo) rows of ld_p elements.
__device__ __forceinline__ float load_feat(const float* p) { return __ldg(p); }
__device__ __forceinline__ float load_feat(const __nv_bfloat16* p) { return __bfloat162float(__ldg(p)); }

template <int D, int KP, int CPL, class BASIS, class ARGS, class FT>
__global__ void __launch_bounds__(conv_warps<KP>() * 32)
project_kernel(ARGS args, int K, const float* __restrict__ pts, const FT* __restrict__ feats, int cin,
               const float* __restrict__ samples, const int2* __restrict__ neighbors,
               const int32_t* __restrict__ start_ids, const float* __restrict__ radii, int m_begin, int m_end,
               __nv_bfloat16* __restrict__ p_hi, __nv_bfloat16* __restrict__ p_lo, int ld_p) {
    // CPL = channels per lane: at most 64 / KP, fewer when Cin does not fill 32 * CPL channels
    constexpr int kConvWarps = conv_warps<KP>();
    __shared__ float s_params[BASIS::kParamFloats];
    // rows of KP + 4 floats: 16-byte aligned, and 128-bit stores of 8 consecutive lanes hit distinct banks
    __shared__ __align__(16) float s_basis[kConvWarps][32][KP + 4];
    __shared__ int s_n0[kConvWarps][32];
    BASIS::load_params(s_params, args, K);
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = lane_id();
    float inv[D];
#pragma unroll
    for (int d = 0; d < D; ++d) inv[d] = BASIS::kUsesOffset ? __frcp_rn(__ldg(radii + d)) : 0.f;
    const int inner = cin * K;

    for (int m = m_begin + blockIdx.x * kConvWarps + warp; m < m_end; m += gridDim.x * kConvWarps) {
        const int lo = (m > 0) ? __ldg(start_ids + m - 1) : 0;
        const int hi = __ldg(start_ids + m);
        float s[D];
#pragma unroll
        for (int d = 0; d < D; ++d) s[d] = BASIS::kUsesOffset ? __ldg(samples + (int64_t)m * D + d) : 0.f;
        const size_t row = (size_t)(m - m_begin) * ld_p;

        for (int cb = 0; cb < cin; cb += 32 * CPL) {
            float acc[CPL][KP];
#pragma unroll
            for (int i = 0; i < CPL; ++i)
#pragma unroll
                for (int k = 0; k < KP; ++k) acc[i][k] = 0.f;

            for (int t0 = lo; t0 < hi; t0 += 32) {
                // Lanes as neighbors: offset and basis row of pair t0 + lane.
                const int t = t0 + lane;
                if (t < hi) {
                    const int n0 = __ldg(&neighbors[t]).x;
                    float d[D], b[KP];
#pragma unroll
                    for (int x = 0; x < D; ++x) d[x] = BASIS::kUsesOffset ? (__ldg(pts + (int64_t)n0 * D + x) - s[x]) * inv[x] : 0.f;
                    BASIS::eval(s_params, args, K, d, n0, t, m, b);
#pragma unroll
                    for (int k = 0; k < KP; k += 4)
                        *reinterpret_cast<float4*>(&s_basis[warp][lane][k]) = make_float4(b[k], b[k + 1], b[k + 2], b[k + 3]);
                    s_n0[warp][lane] = n0;
                }
                __syncwarp();
                // Lanes as channels: stream the feature rows of the staged neighbors, four neighbors
                // per step so that 4 * CPL independent loads are in flight before the FMAs need them.
                const int cnt = min(32, hi - t0);
                // Software pipeline: the loads of the next four neighbors are issued before the FMAs
                // of the current four, so L2 latency overlaps the arithmetic inside one warp.
                auto load4 = [&](int j0, float (&f)[4][CPL]) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int j = min(j0 + u, cnt - 1);
                        const FT* frow = feats + (int64_t)s_n0[warp][j] * cin + cb + lane;
#pragma unroll
                        for (int i = 0; i < CPL; ++i)
                            f[u][i] = (j0 + u < cnt && cb + i * 32 + lane < cin) ? load_feat(frow + i * 32) : 0.f;
                    }
                };
                float fa[4][CPL], fb[4][CPL];
                load4(0, fa);
                for (int j0 = 0; j0 < cnt; j0 += 8) {
                    if (j0 + 4 < cnt) load4(j0 + 4, fb);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int j = min(j0 + u, cnt - 1);
#pragma unroll
                        for (int k = 0; k < KP; k += 4) {
                            const float4 b4 = *reinterpret_cast<const float4*>(&s_basis[warp][j][k]);
                            const float bk[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
                            for (int q = 0; q < 4; ++q)
#pragma unroll
                                for (int i = 0; i < CPL; ++i) acc[i][k + q] = fmaf(fa[u][i], bk[q], acc[i][k + q]);
                        }
                    }
                    if (j0 + 4 >= cnt) break;
                    if (j0 + 8 < cnt) load4(j0 + 8, fa);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int j = min(j0 + 4 + u, cnt - 1);
#pragma unroll
                        for (int k = 0; k < KP; k += 4) {
                            const float4 b4 = *reinterpret_cast<const float4*>(&s_basis[warp][j][k]);
                            const float bk[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
                            for (int q = 0; q < 4; ++q)
#pragma unroll
                                for (int i = 0; i < CPL; ++i) acc[i][k + q] = fmaf(fb[u][i], bk[q], acc[i][k + q]);
                        }
                    }
                }
                __syncwarp();
            }
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                const int c = cb + i * 32 + lane;
                if (c < cin) {
                    if (K == KP && (KP % 8) == 0) {
                        // K bf16 values of one channel are contiguous and 16-byte aligned: 128-bit stores
                        // (a 2-byte store per value would cost one memory transaction each).
#pragma unroll
                        for (int k = 0; k < KP; k += 8) {
                            uint32_t hw[4], lw[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const float v0 = acc[i][k + 2 * q], v1 = acc[i][k + 2 * q + 1];
                                const __nv_bfloat162 h2 = __floats2bfloat162_rn(v0, v1);
                                const __nv_bfloat162 l2 = __floats2bfloat162_rn(v0 - __low2float(h2), v1 - __high2float(h2));
                                hw[q] = *reinterpret_cast<const uint32_t*>(&h2);
                                lw[q] = *reinterpret_cast<const uint32_t*>(&l2);
                            }
                            *reinterpret_cast<uint4*>(p_hi + row + (size_t)c * K + k) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                            if (p_lo)
                                *reinterpret_cast<uint4*>(p_lo + row + (size_t)c * K + k) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < KP; ++k) {
                            if (k < K) {
                                const float v = acc[i][k];
                                const __nv_bfloat16 h = __float2bfloat16_rn(v);
                                p_hi[row + (size_t)c * K + k] = h;
                                if (p_lo) p_lo[row + (size_t)c * K + k] = __float2bfloat16_rn(v - __bfloat162float(h));
                            }
                        }
                    }
                }
            }
        }
        // Padding columns feed the tensor cores too: keep them zero.
        for (int c = inner + lane; c < ld_p; c += 32) {
            p_hi[row + c] = __float2bfloat16_rn(0.f);
            if (p_lo) p_lo[row + c] = __float2bfloat16_rn(0.f);
        }
    }
}

// Sum over the 32 lanes of a KP-vector held by every lane.  Recursive halving: at each step a
// lane hands half of its entries to its partner, so 32 lanes end up owning the KP sums between
// them (entries [k0, k0 + n) on return; lanes that share entries hold identical sums).
template <int KP>
__device__ __forceinline__ void warp_reduce_scatter(float (&v)[KP], int lane, int& k0, int& n) {
    n = KP;
    k0 = 0;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        if (n > 1) {
            n >>= 1;
            const bool up = (lane & off) != 0;
#pragma unroll
            for (int q = 0; q < KP / 2; ++q) {
                if (q < n) {
                    const float send = up ? v[q] : v[q + n];
                    const float keep = up ? v[q + n] : v[q];
                    v[q] = keep + __shfl_xor_sync(kFullMask, send, off);
                }
            }
            k0 += up ? n : 0;
        } else {
            v[0] += __shfl_xor_sync(kFullMask, v[0], off);
        }
    }
}

// Projection for narrow inputs (Cin * KP <= 64, e.g. the xyz or constant features of a first
// layer).  With lanes as channels almost every lane would idle; here the lanes stay neighbors for
// the whole sample: each accumulates its own pairs' f[c] * b[k] products for ALL (c, k) in
// registers, and one reduce-scatter over the warp leaves every lane with two finished entries of
// the sample's P row, which is then written with one coalesced store per plane.
template <int D, int KP, class BASIS, class ARGS, class FT>
__global__ void __launch_bounds__(128)
project_narrow_kernel(ARGS args, int K, const float* __restrict__ pts, const FT* __restrict__ feats, int cin,
                      const float* __restrict__ samples, const int2* __restrict__ neighbors,
                      const int32_t* __restrict__ start_ids, const float* __restrict__ radii, int m_begin, int m_end,
                      __nv_bfloat16* __restrict__ p_hi, __nv_bfloat16* __restrict__ p_lo, int ld_p) {
    constexpr int CS = 64 / KP;  // channel slots
    __shared__ float s_params[BASIS::kParamFloats];
    BASIS::load_params(s_params, args, K);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = lane_id();
    float inv[D];
#pragma unroll
    for (int d = 0; d < D; ++d) inv[d] = BASIS::kUsesOffset ? __frcp_rn(__ldg(radii + d)) : 0.f;
    const int inner = cin * K;

    for (int m = m_begin + blockIdx.x * 4 + warp; m < m_end; m += gridDim.x * 4) {
        const int lo = (m > 0) ? __ldg(start_ids + m - 1) : 0;
        const int hi = __ldg(start_ids + m);
        float s[D];
#pragma unroll
        for (int d = 0; d < D; ++d) s[d] = BASIS::kUsesOffset ? __ldg(samples + (int64_t)m * D + d) : 0.f;
        float acc[64];
#pragma unroll
        for (int e = 0; e < 64; ++e) acc[e] = 0.f;
        for (int t = lo + lane; t < hi; t += 32) {
            const int n0 = __ldg(&neighbors[t]).x;
            float d[D], b[KP], f[CS];
#pragma unroll
            for (int c = 0; c < CS; ++c) f[c] = (c < cin) ? load_feat(feats + (int64_t)n0 * cin + c) : 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) d[x] = BASIS::kUsesOffset ? (__ldg(pts + (int64_t)n0 * D + x) - s[x]) * inv[x] : 0.f;
            BASIS::eval(s_params, args, K, d, n0, t, m, b);
#pragma unroll
            for (int c = 0; c < CS; ++c)
#pragma unroll
                for (int k = 0; k < KP; ++k) acc[c * KP + k] = fmaf(f[c], b[k], acc[c * KP + k]);
        }
        int e0, n;
        warp_reduce_scatter<64>(acc, lane, e0, n);  // n == 2: this lane owns entries e0 and e0 + 1 (c = e / KP, k = e % KP)
        const size_t row = (size_t)(m - m_begin) * ld_p;
        if (K == KP) {
            // entry e sits at column e; columns past Cin * K up to ld_p (= 64) are the zero slots c >= Cin
            const float v0 = acc[0], v1 = acc[1];
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(v0, v1);
            *reinterpret_cast<__nv_bfloat162*>(p_hi + row + e0) = h2;
            if (p_lo)
                *reinterpret_cast<__nv_bfloat162*>(p_lo + row + e0) =
                    __floats2bfloat162_rn(v0 - __low2float(h2), v1 - __high2float(h2));
        } else {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int e = e0 + q, c = e / KP, k = e - c * KP;
                if (c < cin && k < K) {
                    const float v = acc[q];
                    const __nv_bfloat16 h = __float2bfloat16_rn(v);
                    p_hi[row + (size_t)c * K + k] = h;
                    if (p_lo) p_lo[row + (size_t)c * K + k] = __float2bfloat16_rn(v - __bfloat162float(h));
                }
            }
            for (int c = inner + lane; c < ld_p; c += 32) {
                p_hi[row + c] = __float2bfloat16_rn(0.f);
                if (p_lo) p_lo[row + c] = __float2bfloat16_rn(0.f);
            }
        }
    }
}

// Everything of the backward pass that runs per neighbor pair, given dP = g W^T for the samples
// [m_begin, m_end) (pccnn_lib_ops/pcconvs/shared/feat_basis_proj_grads.cu:32-154, then the basis
// and offset gradients of kernel_pts_basis.cu:41-70 / mlp_basis.cu:50-96 and pt_diff.cu:51-80 of
// the reference, which are ~15 separate launches there):
//     dF[n0, c]  += sum_k dP[m, c, k] * b[t, k]
//     db[t, k]    = sum_c dP[m, c, k] * F[n0, c]   -> basis gradient -> d(offset) and parameter gradients
//     dPts[n0]   += d(offset) / radii,   dSamples[m] = -sum_t d(offset) / radii
// A warp owns a sample.  The lanes alternate between "32 neighbors" (basis, basis gradient) and
// "32 channels x CPL" (the two contractions against the sample's dP row held in registers).
template <int D, int KP, int CPL, class BASIS, class ARGS>
__global__ void __launch_bounds__(conv_warps<KP>() * 32)
backward_pairs_kernel(ARGS args, int K, const float* __restrict__ pts, const float* __restrict__ feats, int cin,
                      const float* __restrict__ samples, const int2* __restrict__ neighbors,
                      const int32_t* __restrict__ start_ids, const float* __restrict__ radii, int m_begin, int m_end,
                      const float* __restrict__ d_proj, float* __restrict__ d_feat, float* __restrict__ d_pts,
                      float* __restrict__ d_samples, float* __restrict__ d_param0, float* __restrict__ d_param1,
                      float* __restrict__ d_pdf) {
    constexpr int kConvWarps = conv_warps<KP>();
    __shared__ float s_params[BASIS::kParamFloats];
    __shared__ float s_grad[BASIS::kGradFloats];
    __shared__ __align__(16) float s_basis[kConvWarps][32][KP + 4];
    __shared__ float s_db[kConvWarps][32][KP + 1];
    __shared__ int s_n0[kConvWarps][32];
    BASIS::load_params(s_params, args, K);
    for (int i = threadIdx.x; i < BASIS::kGradFloats; i += blockDim.x) s_grad[i] = 0.f;
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = lane_id();
    float inv[D];
#pragma unroll
    for (int d = 0; d < D; ++d) inv[d] = BASIS::kUsesOffset ? __frcp_rn(__ldg(radii + d)) : 0.f;
    const int inner = cin * K;

    for (int m = m_begin + blockIdx.x * kConvWarps + warp; m < m_end; m += gridDim.x * kConvWarps) {
        const int lo = (m > 0) ? __ldg(start_ids + m - 1) : 0;
        const int hi = __ldg(start_ids + m);
        float s[D], ds_acc[D];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            s[d] = BASIS::kUsesOffset ? __ldg(samples + (int64_t)m * D + d) : 0.f;
            ds_acc[d] = 0.f;
        }
        const float* grow = d_proj + (size_t)(m - m_begin) * inner;

        for (int t0 = lo; t0 < hi; t0 += 32) {
            // Lanes as neighbors: offset and basis row of pair t0 + lane (kept for the gradient below).
            const int t = t0 + lane;
            int n0 = 0;
            float d[D];
#pragma unroll
            for (int x = 0; x < D; ++x) d[x] = 0.f;
            if (t < hi) {
                n0 = __ldg(&neighbors[t]).x;
                float b[KP];
#pragma unroll
                for (int x = 0; x < D; ++x) d[x] = BASIS::kUsesOffset ? (__ldg(pts + (int64_t)n0 * D + x) - s[x]) * inv[x] : 0.f;
                BASIS::eval(s_params, args, K, d, n0, t, m, b);
#pragma unroll
                for (int k = 0; k < KP; k += 4)
                    *reinterpret_cast<float4*>(&s_basis[warp][lane][k]) = make_float4(b[k], b[k + 1], b[k + 2], b[k + 3]);
                s_n0[warp][lane] = n0;
            }
#pragma unroll
            for (int k = 0; k < KP; ++k) s_db[warp][lane][k] = 0.f;
            __syncwarp();

            // Lanes as channels.
            const int cnt = min(32, hi - t0);
            for (int cb = 0; cb < cin; cb += 32 * CPL) {
                float g[CPL][KP];
#pragma unroll
                for (int i = 0; i < CPL; ++i) {
                    const int c = cb + i * 32 + lane;
                    if (K == KP && (KP % 4) == 0) {
#pragma unroll
                        for (int k = 0; k < KP; k += 4) {
                            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (c < cin) v = __ldg(reinterpret_cast<const float4*>(grow + (size_t)c * K + k));
                            g[i][k] = v.x; g[i][k + 1] = v.y; g[i][k + 2] = v.z; g[i][k + 3] = v.w;
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < KP; ++k) g[i][k] = (c < cin && k < K) ? __ldg(grow + (size_t)c * K + k) : 0.f;
                    }
                }
                // The dP row as fp32x2 pairs (k, k + 1): both contractions below run as packed FMAs, one
                // issue slot for two products, each half rounded like the scalar FMA.
                unsigned long long g2[CPL][KP / 2];
#pragma unroll
                for (int i = 0; i < CPL; ++i)
#pragma unroll
                    for (int k = 0; k < KP; k += 2) g2[i][k / 2] = pack_f32x2(g[i][k], g[i][k + 1]);
                for (int j0 = 0; j0 < cnt; j0 += 2) {
                    float f[2][CPL];
                    int nj[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        nj[u] = s_n0[warp][min(j0 + u, cnt - 1)];
                        const float* frow = feats + (int64_t)nj[u] * cin + cb + lane;
#pragma unroll
                        for (int i = 0; i < CPL; ++i)
                            f[u][i] = (j0 + u < cnt && cb + i * 32 + lane < cin) ? __ldg(frow + i * 32) : 0.f;
                    }
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        if (j0 + u >= cnt) break;
                        const int j = j0 + u;
                        float df[CPL], pb[KP];
                        unsigned long long df2[CPL], f2[CPL];  // df2: partial sums over even / odd k
#pragma unroll
                        for (int i = 0; i < CPL; ++i) {
                            df2[i] = 0ull;
                            f2[i] = pack_f32x2(f[u][i], f[u][i]);
                        }
#pragma unroll
                        for (int k = 0; k < KP; k += 4) {
                            const float4 b4 = *reinterpret_cast<const float4*>(&s_basis[warp][j][k]);
                            const unsigned long long bb[2] = {pack_f32x2(b4.x, b4.y), pack_f32x2(b4.z, b4.w)};
#pragma unroll
                            for (int q = 0; q < 2; ++q) {
                                unsigned long long acc2 = 0ull;
#pragma unroll
                                for (int i = 0; i < CPL; ++i) {
                                    df2[i] = fma_f32x2(g2[i][k / 2 + q], bb[q], df2[i]);
                                    acc2 = fma_f32x2(g2[i][k / 2 + q], f2[i], acc2);
                                }
                                unpack_f32x2(acc2, pb[k + 2 * q], pb[k + 2 * q + 1]);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < CPL; ++i) {
                            float even, odd;
                            unpack_f32x2(df2[i], even, odd);
                            df[i] = even + odd;
                        }
#pragma unroll
                        for (int i = 0; i < CPL; ++i) {
                            const int c = cb + i * 32 + lane;
                            if (c < cin && df[i] != 0.f) atomicAdd(d_feat + (int64_t)nj[u] * cin + c, df[i]);
                        }
                        int k0, n;
                        warp_reduce_scatter<KP>(pb, lane, k0, n);
                        // lanes whose low bits are zero speak for their group of identical sums
                        if ((lane & ((32 / (KP < 32 ? KP : 32)) - 1)) == 0) {
#pragma unroll
                            for (int q = 0; q < (KP + 31) / 32; ++q) s_db[warp][j][k0 + q] += pb[q];
                        }
                    }
                }
                __syncwarp();
            }

            // Lanes as neighbors again: basis gradient, offset gradient, point gradients.
            float d_off[D], dpdf = 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) d_off[x] = 0.f;
            BASIS::grad(s_params, args, K, d, n0, t, m, t < hi, s_db[warp][lane], d_off, s_grad, dpdf);
            if (t < hi) {
#pragma unroll
                for (int x = 0; x < D; ++x) {
                    const float gx = d_off[x] * inv[x];
                    if (d_pts && gx != 0.f) atomicAdd(d_pts + (int64_t)n0 * D + x, gx);
                    ds_acc[x] += gx;
                }
                if (d_pdf && dpdf != 0.f) atomicAdd(d_pdf + n0, dpdf);
            }
            __syncwarp();
        }
#pragma unroll
        for (int x = 0; x < D; ++x) {
            const float tot = warp_sum(ds_acc[x]);
            if (lane == 0 && d_samples) d_samples[(int64_t)m * D + x] = -tot;
        }
    }
    __syncthreads();
    BASIS::flush(s_grad, K, d_param0, d_param1);
}

template <int D, class ARGS, template <int, int> class BASIS>
static int launch_backward_pairs(int K, const ARGS& args, const float* pts, const float* feats, int cin,
                                 const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                                 const float* radii, int m_begin, int m_end, const float* d_proj, float* d_feat,
                                 float* d_pts, float* d_samples, float* d_param0, float* d_param1, float* d_pdf,
                                 cudaStream_t s) {
    const int count = m_end - m_begin;
    if (count <= 0) return PCCNN_OK;
#define PCCNN_BACKWARD_C(KP, CPL)                                                                                   \
    backward_pairs_kernel<D, KP, CPL, BASIS<D, KP>, ARGS>                                                           \
        <<<grid_for((int64_t)count * 32, conv_warps<KP>() * 32, 4), conv_warps<KP>() * 32, 0, s>>>(                  \
        args, K, pts, feats, cin, samples, (const int2*)neighbors, start_ids, radii, m_begin, m_end, d_proj, d_feat, \
        d_pts, d_samples, d_param0, d_param1, d_pdf)
#define PCCNN_BACKWARD(KP)                                                                                          \
    do {                                                                                                            \
        constexpr int kMax = 64 / KP;                                                                               \
        if (kMax >= 8 && cin > 128) PCCNN_BACKWARD_C(KP, (kMax >= 8 ? 8 : kMax));                                    \
        else if (kMax >= 4 && cin > 64) PCCNN_BACKWARD_C(KP, (kMax >= 4 ? 4 : kMax));                                \
        else if (kMax >= 2 && cin > 32) PCCNN_BACKWARD_C(KP, (kMax >= 2 ? 2 : kMax));                                \
        else PCCNN_BACKWARD_C(KP, 1);                                                                               \
    } while (0)
    if (K <= 8) PCCNN_BACKWARD(8);
    else if (K <= 16) PCCNN_BACKWARD(16);
    else if (K <= 32) PCCNN_BACKWARD(32);
    else PCCNN_BACKWARD(64);
#undef PCCNN_BACKWARD
#undef PCCNN_BACKWARD_C
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

template <int D, class ARGS, template <int, int> class BASIS, class FT = float>
static int launch_project(int K, const ARGS& args, const float* pts, const FT* feats, int cin, const float* samples,
                          const int32_t* neighbors, const int32_t* start_ids, const float* radii, int m_begin,
                          int m_end, void* p_hi, void* p_lo, int ld_p, cudaStream_t s) {
    const int count = m_end - m_begin;
    if (count <= 0) return PCCNN_OK;
    // channels per lane: the largest power of two <= 64 / KP that Cin can still fill
#define PCCNN_PROJECT_C(KP, CPL)                                                                   \
    project_kernel<D, KP, CPL, BASIS<D, KP>, ARGS, FT>                                             \
        <<<grid_for((int64_t)count * 32, conv_warps<KP>() * 32, 8), conv_warps<KP>() * 32, 0, s>>>( \
            args, K, pts, feats, cin, samples, (const int2*)neighbors, start_ids, radii, m_begin,  \
            m_end, (__nv_bfloat16*)p_hi, (__nv_bfloat16*)p_lo, ld_p)
#define PCCNN_PROJECT(KP)                                                        \
    do {                                                                         \
        constexpr int kMax = 64 / KP;                                            \
        if (cin <= kMax)                                                         \
            project_narrow_kernel<D, KP, BASIS<D, KP>, ARGS, FT>                 \
                <<<grid_for((int64_t)count * 32, 128, 8), 128, 0, s>>>(          \
                    args, K, pts, feats, cin, samples, (const int2*)neighbors, start_ids, radii, m_begin, \
                    m_end, (__nv_bfloat16*)p_hi, (__nv_bfloat16*)p_lo, ld_p);     \
        else if (kMax >= 8 && cin > 128) PCCNN_PROJECT_C(KP, (kMax >= 8 ? 8 : kMax)); \
        else if (kMax >= 4 && cin > 64) PCCNN_PROJECT_C(KP, (kMax >= 4 ? 4 : kMax)); \
        else if (kMax >= 2 && cin > 32) PCCNN_PROJECT_C(KP, (kMax >= 2 ? 2 : kMax)); \
        else PCCNN_PROJECT_C(KP, 1);                                             \
    } while (0)
    if (K <= 8) PCCNN_PROJECT(8);
    else if (K <= 16) PCCNN_PROJECT(16);
    else if (K <= 32) PCCNN_PROJECT(32);
    else PCCNN_PROJECT(64);
#undef PCCNN_PROJECT
#undef PCCNN_PROJECT_C
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

// Samples are processed in chunks so that the P scratch stays bounded: 131 072 samples, and 524 288 for calls with
// more samples than that whose P row has at most 2048 entries (a 2 M-point scene is then 4 chunks instead of 16; the
// ends of the chunks' launches, where the SMs run dry one by one, cost 2 % of such a layer; the scratch grows to
// ~9 GB for 128 channels x 16 basis values, and an index into a chunk's P stays below 2^30).
static int64_t conv_chunk(int64_t num_samples, int ld_p) {
    const int64_t small = 1 << 17, large = 1 << 19;
    if (num_samples <= 0) return 1;
    return num_samples < small ? num_samples : ((num_samples > large && ld_p <= 2048) ? large : small);
}

struct ConvLayout {
    int ld_p;      // padded Cin * K
    int ld_f;      // elements per row of the bf16 feature planes (Cin rounded up to 8)
    int64_t chunk;
    size_t p_hi_off, p_lo_off, w_hi_off, w_lo_off, status_off, f_hi_off, f_lo_off, total;
};

// Bytes of one bf16 feature plane [num_pts, ld_f] for the tensor-core pair kernels (0 when they cannot apply).
static size_t feature_plane_bytes(int64_t num_pts, int cin) {
    return cin >= 32 ? align_up((size_t)(num_pts > 0 ? num_pts : 1) * ((cin + 7) / 8 * 8) * 2) : 0;
}

static ConvLayout conv_layout(int64_t num_pts, int64_t num_samples, int cin, int K, int cout) {
    ConvLayout L;
    L.ld_p = (cin * K + 63) / 64 * 64;
    L.chunk = conv_chunk(num_samples, L.ld_p);
    const size_t p_bytes = align_up((size_t)L.chunk * L.ld_p * 2);
    const size_t w_bytes = align_up((size_t)cout * L.ld_p * 2);
    L.p_hi_off = 0;
    L.p_lo_off = p_bytes;
    L.w_hi_off = 2 * p_bytes;
    L.w_lo_off = L.w_hi_off + w_bytes;
    L.status_off = L.w_lo_off + w_bytes;
    L.ld_f = (cin + 7) / 8 * 8;
    L.f_hi_off = L.status_off + 256;
    L.f_lo_off = L.f_hi_off + feature_plane_bytes(num_pts, cin);
    L.total = L.f_lo_off + feature_plane_bytes(num_pts, cin);
    return L;
}

template <class ARGS, template <int, int> class BASIS, bool WITH_BF16 = false>
static int conv_forward(const char* who, int D, int K, const ARGS& args, int64_t num_pts, const float* pts,
                        const void* feats_any, int cin, int64_t num_samples, const float* samples,
                        const int32_t* neighbors, const int32_t* start_ids, const float* radii, int num_mlps,
                        const void* weights_any, int cout, void* out_any, void* workspace, size_t workspace_bytes,
                        cudaStream_t s, bool io_bf16 = false) {
    // io_bf16: features, weights and output are bf16 (inference configuration): one tensor-core pass,
    // P kept as a single bf16 plane, fp32 accumulation.
    const float* feats = (const float*)feats_any;
    const float* weights = (const float*)weights_any;
    float* out = (float*)out_any;
    if (int rc = take_sticky_status(who)) return rc;  // an earlier call's tensor-core kernel gave up
    PCCNN_CHECK_ARG(!io_bf16 || (WITH_BF16 && D == 3), "%s: bf16 features are supported for 3-D KPConv only", who);
    PCCNN_CHECK_ARG(D >= kMinDims && D <= kMaxDims, "%s: point dimension %d outside [2, 6]", who, D);
    PCCNN_CHECK_ARG(K >= 1 && K <= 64, "%s: basis size %d outside [1, 64]", who, K);
    PCCNN_CHECK_ARG(cin >= 1 && cout >= 1 && num_mlps >= 1 && cout % num_mlps == 0 && (cin * K) % num_mlps == 0,
                    "%s: bad channel counts (cin %d, cout %d, mlps %d)", who, cin, cout, num_mlps);
    PCCNN_CHECK_ARG(num_samples >= 0 && num_samples < 0x7fffffffLL && num_pts >= 0, "%s: bad sizes", who);
    // Several MLPs: MLP j reads the j-th slice of the P rows and writes the j-th slice of the outputs; the P
    // slices are TMA operands of their own, so they must start on 16-byte boundaries (8 bf16 values).
    PCCNN_CHECK_ARG(num_mlps == 1 || (cin * K / num_mlps) % 8 == 0,
                    "%s: with several MLPs, Cin*K per MLP must be a multiple of 8", who);
    if (num_samples == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(pts && feats && samples && start_ids && radii && weights && out, "%s: null pointer", who);
    const ConvLayout L = conv_layout(num_pts, num_samples, cin, K, cout);
    if (!workspace || workspace_bytes < L.total) {
        set_error("%s: workspace of %zu bytes, need %zu", who, workspace_bytes, L.total);
        return PCCNN_ERR_WORKSPACE;
    }
    char* ws = (char*)workspace;
    int* status = (int*)(ws + L.status_off);
    PCCNN_CUDA(cudaMemsetAsync(status, 0, 4, s));

    // W^T as bf16 hi/lo, K-contiguous.  With several MLPs the weight tensor is [mlps, inner/mlps... ]:
    // MLP j maps the j-th slice of the flattened (c, k) index to the j-th slice of the outputs
    // (mcconv.cu:59-68 of the reference reshapes exactly so).
    const int inner = cin * K, inner_j = inner / num_mlps, cout_j = cout / num_mlps;
    PCCNN_CUDA(cudaMemsetAsync(ws + L.w_hi_off, 0, L.status_off - L.w_hi_off, s));
    for (int j = 0; j < num_mlps; ++j) {
        const size_t off = (size_t)j * cout_j * L.ld_p * 2;
        int rc;
        if (io_bf16)
            rc = transpose_bf16(inner_j, cout_j, (const __nv_bfloat16*)weights_any + (size_t)j * inner_j * cout_j, cout_j,
                                L.ld_p, ws + L.w_hi_off + off, s);
        else
            rc = split_bf16_transpose(inner_j, cout_j, weights + (size_t)j * inner_j * cout_j, cout_j, L.ld_p,
                                      ws + L.w_hi_off + off, ws + L.w_lo_off + off, s);
        if (rc) return rc;
    }
    const bool tc = use_tensor_core_pairs(D, cin) && (!io_bf16 || cin % 8 == 0);
    FeaturePlanes planes{(const __nv_bfloat16*)(ws + L.f_hi_off), (const __nv_bfloat16*)(ws + L.f_lo_off), L.ld_f};
    if (tc && io_bf16) planes = FeaturePlanes{(const __nv_bfloat16*)feats_any, nullptr, cin};  // used as they are
    if (tc && !io_bf16)
        if (int rc = split_features(num_pts, cin, feats, ws + L.f_hi_off, ws + L.f_lo_off, s)) return rc;
    for (int64_t m0 = 0; m0 < num_samples; m0 += L.chunk) {
        const int64_t m1 = (m0 + L.chunk < num_samples) ? m0 + L.chunk : num_samples;
        int rc = PCCNN_OK;
        if (io_bf16) {
            if constexpr (WITH_BF16) {  // only the operators that offer the bf16 path instantiate its kernels
                if (tc)
                    rc = launch_project_tc<ARGS, BASIS, false>(K, args, pts, planes, cin, samples, neighbors, start_ids, radii,
                                                               (int)m0, (int)m1, ws + L.p_hi_off, nullptr, L.ld_p, status, s);
                else
                    rc = launch_project<3, ARGS, BASIS, __nv_bfloat16>(K, args, pts, (const __nv_bfloat16*)feats_any, cin,
                                                                       samples, neighbors, start_ids, radii, (int)m0,
                                                                       (int)m1, ws + L.p_hi_off, nullptr, L.ld_p, s);
            }
        } else if (tc) {
            rc = launch_project_tc<ARGS, BASIS, true>(K, args, pts, planes, cin, samples, neighbors, start_ids, radii, (int)m0,
                                                      (int)m1, ws + L.p_hi_off, ws + L.p_lo_off, L.ld_p, status, s);
        } else {
            rc = dispatch_dims<BasisTraits<BASIS>::kOnly3D>(D, [&](auto dim) {
            constexpr int DIM = decltype(dim)::value;
            return launch_project<DIM, ARGS, BASIS>(K, args, pts, feats, cin, samples, neighbors,
                                                                         start_ids, radii, (int)m0, (int)m1,
                                                                         ws + L.p_hi_off, ws + L.p_lo_off, L.ld_p, s);
        });
        }
        if (rc) return rc;
        for (int j = 0; j < num_mlps; ++j) {
            // Slice j of the P rows (offset j * inner_j, 16-byte aligned: inner_j % 8 == 0 was checked above)
            // times W_j^T.  The reduction runs over the slice rounded up to 64 columns: what is read past the
            // slice (the next MLP's columns, or the zero fill past the row end) meets the zero padding of W_j^T.
            const size_t a_off = (size_t)j * inner_j * 2;
            const size_t b_off = (size_t)j * cout_j * L.ld_p * 2;
            const int kp = num_mlps == 1 ? L.ld_p : (inner_j + 63) / 64 * 64;
            GemmOperand a{ws + L.p_hi_off + a_off, io_bf16 ? nullptr : ws + L.p_lo_off + a_off, L.ld_p,
                          L.ld_p - (int64_t)j * inner_j};
            GemmOperand b{ws + L.w_hi_off + b_off, io_bf16 ? nullptr : ws + L.w_lo_off + b_off, L.ld_p};
            float* c_ptr = io_bf16 ? (float*)((__nv_bfloat16*)out_any + (size_t)m0 * cout + (size_t)j * cout_j)
                                   : out + (size_t)m0 * cout + (size_t)j * cout_j;
            if (int rc2 = gemm_bf16_nt(a, b, c_ptr, m1 - m0, cout_j, kp, cout, status, s, io_bf16 ? 1 : 0)) return rc2;
        }
    }
    return publish_status(status, kOriginConvForward, s);
}

// ---- forward without a neighbor list ------------------------------------------------------------------------
struct ConvGridLayout {
    ConvLayout base;
    size_t f_hi_off, f_lo_off, total;
};

static ConvGridLayout conv_grid_layout(int64_t num_pts, int64_t num_samples, int cin, int K, int cout) {
    ConvGridLayout G;
    G.base = conv_layout(0, num_samples, cin, K, cout);  // the planes of the list-based path are not needed
    const size_t plane = align_up((size_t)(num_pts > 0 ? num_pts : 1) * ((cin + 7) / 8 * 8) * 2);
    G.f_hi_off = G.base.f_hi_off;
    G.f_lo_off = G.f_hi_off + plane;
    G.total = G.f_lo_off + plane;
    return G;
}

// out = P W with P from project_tc_grid_kernel: the neighbors are found on the grid inside the projection, no list.
// Points, keys and table as the search takes them (grid order); `pt_index_map` (may be null = identity) maps a sorted
// position to the row of `feats`, which are in the caller's order.  3-D points.
template <class ARGS, template <int, int> class BASIS>
static int conv_forward_grid(const char* who, int K, const ARGS& args, int64_t num_pts, const float* sorted_pts,
                             const int64_t* sorted_keys, const int64_t* pt_index_map, const void* feats_any, int io_bf16,
                             int cin, int64_t num_samples, const float* samples, const int64_t* sample_keys,
                             const int32_t* grid_ds, const int32_t* grid_size, const float* radii, const void* weights_any,
                             int cout, void* out_any, void* workspace, size_t workspace_bytes, cudaStream_t s) {
    if (int rc = take_sticky_status(who)) return rc;
    PCCNN_CHECK_ARG(K >= 1 && K <= 64, "%s: basis size %d outside [1, 64]", who, K);
    PCCNN_CHECK_ARG(cin >= 1 && cout >= 1, "%s: bad channel counts (cin %d, cout %d)", who, cin, cout);
    PCCNN_CHECK_ARG(num_samples >= 0 && num_samples < 0x7fffffffLL && num_pts >= 0 && num_pts < 0x7fffffffLL, "%s: bad sizes", who);
    if (num_samples == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(samples && sample_keys && grid_ds && grid_size && radii && weights_any && out_any, "%s: null pointer", who);
    PCCNN_CHECK_ARG(num_pts == 0 || (sorted_pts && sorted_keys && feats_any), "%s: null points", who);
    const ConvGridLayout G = conv_grid_layout(num_pts, num_samples, cin, K, cout);
    const ConvLayout& L = G.base;
    if (!workspace || workspace_bytes < G.total) {
        set_error("%s: workspace of %zu bytes, need %zu", who, workspace_bytes, G.total);
        return PCCNN_ERR_WORKSPACE;
    }
    char* ws = (char*)workspace;
    int* status = (int*)(ws + L.status_off);
    PCCNN_CUDA(cudaMemsetAsync(status, 0, 4, s));
    PCCNN_CUDA(cudaMemsetAsync(ws + L.w_hi_off, 0, L.status_off - L.w_hi_off, s));
    const int inner = cin * K;
    int rc;
    if (io_bf16)
        rc = transpose_bf16(inner, cout, weights_any, cout, L.ld_p, ws + L.w_hi_off, s);
    else
        rc = split_bf16_transpose(inner, cout, (const float*)weights_any, cout, L.ld_p, ws + L.w_hi_off, ws + L.w_lo_off, s);
    if (rc) return rc;
    // feature planes in grid order
    __nv_bfloat16* f_hi = (__nv_bfloat16*)(ws + G.f_hi_off);
    __nv_bfloat16* f_lo = io_bf16 ? nullptr : (__nv_bfloat16*)(ws + G.f_lo_off);
    if (num_pts > 0) {
        const unsigned grid = grid_for(num_pts * (L.ld_f / 8), 256, 8);
        if (io_bf16)
            permute_features_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(num_pts, cin, L.ld_f, (const __nv_bfloat16*)feats_any,
                                                                         pt_index_map, f_hi, f_lo);
        else
            permute_features_kernel<float><<<grid, 256, 0, s>>>(num_pts, cin, L.ld_f, (const float*)feats_any, pt_index_map,
                                                                f_hi, f_lo);
        PCCNN_LAUNCH_CHECK();
    }
    const FeaturePlanes planes{f_hi, f_lo, L.ld_f};
    for (int64_t m0 = 0; m0 < num_samples; m0 += L.chunk) {
        const int64_t m1 = (m0 + L.chunk < num_samples) ? m0 + L.chunk : num_samples;
        if (io_bf16)
            rc = launch_project_tc_grid<ARGS, BASIS, false>(K, args, (int)num_pts, sorted_pts, sorted_keys, planes, cin,
                                                            (int)num_samples, samples, sample_keys, grid_ds, grid_size, radii,
                                                            (int)m0, (int)m1, ws + L.p_hi_off, nullptr, L.ld_p, status, s);
        else
            rc = launch_project_tc_grid<ARGS, BASIS, true>(K, args, (int)num_pts, sorted_pts, sorted_keys, planes, cin,
                                                           (int)num_samples, samples, sample_keys, grid_ds, grid_size, radii,
                                                           (int)m0, (int)m1, ws + L.p_hi_off, ws + L.p_lo_off, L.ld_p, status, s);
        if (rc) return rc;
        GemmOperand a{ws + L.p_hi_off, io_bf16 ? nullptr : ws + L.p_lo_off, L.ld_p};
        GemmOperand b{ws + L.w_hi_off, io_bf16 ? nullptr : ws + L.w_lo_off, L.ld_p};
        float* c_ptr = io_bf16 ? (float*)((__nv_bfloat16*)out_any + (size_t)m0 * cout) : (float*)out_any + (size_t)m0 * cout;
        if ((rc = gemm_bf16_nt(a, b, c_ptr, m1 - m0, cout, L.ld_p, cout, status, s, io_bf16 ? 1 : 0))) return rc;
    }
    return publish_status(status, kOriginConvForward, s);
}

struct ConvBackwardLayout {
    int ld_p, ld_g;
    int64_t chunk;
    int ld_f;
    size_t p_hi_off, p_lo_off, g_hi_off, g_lo_off, dproj_off, w_hi_off, w_lo_off, status_off, f_hi_off, f_lo_off, total;
};

static ConvBackwardLayout conv_backward_layout(int64_t num_pts, int64_t num_samples, int cin, int K, int cout) {
    ConvBackwardLayout L;
    const int inner = cin * K;
    L.ld_p = (inner + 63) / 64 * 64;
    L.ld_g = (cout + 63) / 64 * 64;
    L.chunk = conv_chunk(num_samples, L.ld_p);
    const size_t p_bytes = align_up((size_t)L.chunk * L.ld_p * 2);
    const size_t g_bytes = align_up((size_t)L.chunk * L.ld_g * 2);
    const size_t d_bytes = align_up((size_t)L.chunk * inner * 4);
    const size_t w_bytes = align_up((size_t)inner * L.ld_g * 2);
    L.p_hi_off = 0;
    L.p_lo_off = p_bytes;
    L.g_hi_off = 2 * p_bytes;
    L.g_lo_off = L.g_hi_off + g_bytes;
    L.dproj_off = L.g_lo_off + g_bytes;
    L.w_hi_off = L.dproj_off + d_bytes;
    L.w_lo_off = L.w_hi_off + w_bytes;
    L.status_off = L.w_lo_off + w_bytes;
    L.ld_f = (cin + 7) / 8 * 8;
    L.f_hi_off = L.status_off + 256;
    L.f_lo_off = L.f_hi_off + feature_plane_bytes(num_pts, cin);
    L.total = L.f_lo_off + feature_plane_bytes(num_pts, cin);
    return L;
}

// Event that the next conv_backward of this thread records on its stream as soon as the weight gradient is
// complete (after the last chunk's dW contraction, before that chunk's per-pair kernel), so that a caller can start
// the allreduce of dW on another stream while the rest of the backward pass still runs.  One shot.
extern thread_local cudaEvent_t g_weight_grads_event;  // defined in conv.cu

// Backward of conv_forward.  Per chunk of samples: recompute P, dW += P^T g and dP = g W^T on the
// tensor cores, then the per-pair kernel.  All outputs are zeroed here and accumulated into.
template <class ARGS, template <int, int> class BASIS>
static int conv_backward(const char* who, int D, int K, const ARGS& args, int64_t num_pts, const float* pts,
                         const float* feats, int cin, int64_t num_samples, const float* samples,
                         const int32_t* neighbors, const int32_t* start_ids, const float* radii, int num_mlps,
                         const float* weights, int cout, const float* in_grads, float* d_weights, float* d_feat,
                         float* d_param0, size_t param0_floats, float* d_param1, size_t param1_floats, float* d_pdf,
                         float* d_pts, float* d_samples, void* workspace, size_t workspace_bytes, cudaStream_t s) {
    if (int rc = take_sticky_status(who)) return rc;  // an earlier call's tensor-core kernel gave up
    PCCNN_CHECK_ARG(D >= kMinDims && D <= kMaxDims, "%s: point dimension %d outside [2, 6]", who, D);
    PCCNN_CHECK_ARG(K >= 1 && K <= 64, "%s: basis size %d outside [1, 64]", who, K);
    PCCNN_CHECK_ARG(cin >= 1 && cout >= 1 && num_mlps >= 1 && cout % num_mlps == 0 && (cin * K) % num_mlps == 0,
                    "%s: bad channel counts (cin %d, cout %d, mlps %d)", who, cin, cout, num_mlps);
    PCCNN_CHECK_ARG(num_samples >= 0 && num_samples < 0x7fffffffLL && num_pts >= 0, "%s: bad sizes", who);
    PCCNN_CHECK_ARG(d_weights && d_feat, "%s: null output", who);
    const int inner = cin * K, inner_j = inner / num_mlps, cout_j = cout / num_mlps;
    PCCNN_CHECK_ARG(num_mlps == 1 || (inner_j % 8 == 0 && cout_j % 8 == 0),
                    "%s: with several MLPs, Cin*K per MLP and Cout per MLP must be multiples of 8 (the slices of the "
                    "projected operand and of the upstream gradient are tensor-core operands of their own)", who);
    PCCNN_CUDA(cudaMemsetAsync(d_weights, 0, (size_t)inner * cout_j * 4, s));
    PCCNN_CUDA(cudaMemsetAsync(d_feat, 0, (size_t)num_pts * cin * 4, s));
    if (d_param0) PCCNN_CUDA(cudaMemsetAsync(d_param0, 0, param0_floats * 4, s));
    if (d_param1) PCCNN_CUDA(cudaMemsetAsync(d_param1, 0, param1_floats * 4, s));
    if (d_pdf) PCCNN_CUDA(cudaMemsetAsync(d_pdf, 0, (size_t)num_pts * 4, s));
    if (d_pts) PCCNN_CUDA(cudaMemsetAsync(d_pts, 0, (size_t)num_pts * D * 4, s));
    if (d_samples) PCCNN_CUDA(cudaMemsetAsync(d_samples, 0, (size_t)num_samples * D * 4, s));
    if (num_samples == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(pts && feats && samples && start_ids && radii && weights && in_grads, "%s: null pointer", who);
    const ConvBackwardLayout L = conv_backward_layout(num_pts, num_samples, cin, K, cout);
    if (!workspace || workspace_bytes < L.total) {
        set_error("%s: workspace of %zu bytes, need %zu", who, workspace_bytes, L.total);
        return PCCNN_ERR_WORKSPACE;
    }
    char* ws = (char*)workspace;
    int* status = (int*)(ws + L.status_off);
    PCCNN_CUDA(cudaMemsetAsync(status, 0, 4, s));
    const cudaEvent_t weight_grads_event = g_weight_grads_event;
    g_weight_grads_event = nullptr;
    // W_j as bf16 hi/lo rows [inner_j, ld_g] (reduction index of dP = g W^T is the output channel).
    for (int j = 0; j < num_mlps; ++j) {
        const size_t off = (size_t)j * inner_j * L.ld_g * 2;
        if (int rc = split_bf16(inner_j, cout_j, weights + (size_t)j * inner_j * cout_j, cout_j, L.ld_g,
                                ws + L.w_hi_off + off, ws + L.w_lo_off + off, s))
            return rc;
    }
    float* d_proj = (float*)(ws + L.dproj_off);
    const bool tc = use_tensor_core_pairs(D, cin);
    const FeaturePlanes planes{(const __nv_bfloat16*)(ws + L.f_hi_off), (const __nv_bfloat16*)(ws + L.f_lo_off), L.ld_f};
    if (tc)
        if (int rc = split_features(num_pts, cin, feats, ws + L.f_hi_off, ws + L.f_lo_off, s)) return rc;
    // The tensor-core pair kernel also produces the projected features of its samples when one pass covers all
    // channels (the gathered tile is the same); then the weight-gradient contraction follows it.
    const bool fused_p = tc && cin <= kTcChan;
    for (int64_t m0 = 0; m0 < num_samples; m0 += L.chunk) {
        const int64_t m1 = (m0 + L.chunk < num_samples) ? m0 + L.chunk : num_samples;
        const int64_t rows = m1 - m0;
        int rc = PCCNN_OK;
        if (tc && !fused_p)
            rc = launch_project_tc<ARGS, BASIS, true>(K, args, pts, planes, cin, samples, neighbors, start_ids, radii, (int)m0,
                                                      (int)m1, ws + L.p_hi_off, ws + L.p_lo_off, L.ld_p, status, s);
        else if (!tc)
            rc = dispatch_dims<BasisTraits<BASIS>::kOnly3D>(D, [&](auto dim) {
                constexpr int DIM = decltype(dim)::value;
                return launch_project<DIM, ARGS, BASIS>(K, args, pts, feats, cin, samples, neighbors, start_ids, radii,
                                                        (int)m0, (int)m1, ws + L.p_hi_off, ws + L.p_lo_off, L.ld_p, s);
            });
        if (rc) return rc;
        if ((rc = split_bf16(rows, cout, in_grads + (size_t)m0 * cout, cout, L.ld_g, ws + L.g_hi_off, ws + L.g_lo_off, s)))
            return rc;
        auto operands = [&](int j, GemmOperand& p, GemmOperand& g, GemmOperand& w) {
            p = GemmOperand{ws + L.p_hi_off + (size_t)j * inner_j * 2, ws + L.p_lo_off + (size_t)j * inner_j * 2, L.ld_p,
                            L.ld_p - (int64_t)j * inner_j};
            g = GemmOperand{ws + L.g_hi_off + (size_t)j * cout_j * 2, ws + L.g_lo_off + (size_t)j * cout_j * 2, L.ld_g,
                            L.ld_g - (int64_t)j * cout_j};
            w = GemmOperand{ws + L.w_hi_off + (size_t)j * inner_j * L.ld_g * 2, ws + L.w_lo_off + (size_t)j * inner_j * L.ld_g * 2,
                            L.ld_g};
        };
        auto weight_grads = [&]() -> int {  // dW_j += P_j^T g_j
            for (int j = 0; j < num_mlps; ++j) {
                GemmOperand p, g, w;
                operands(j, p, g, w);
                if (int rc2 = gemm_bf16_tn_accumulate(p, g, d_weights + (size_t)j * inner_j * cout_j, rows, inner_j, cout_j,
                                                      cout_j, status, s))
                    return rc2;
            }
            if (m1 == num_samples && weight_grads_event) PCCNN_CUDA(cudaEventRecord(weight_grads_event, s));  // dW is final
            return PCCNN_OK;
        };
        if (!fused_p)
            if ((rc = weight_grads())) return rc;
        for (int j = 0; j < num_mlps; ++j) {
            GemmOperand p, g, w;
            operands(j, p, g, w);
            // dP_j = g_j W_j^T  ->  columns [j * inner_j, (j + 1) * inner_j) of the dP rows
            // (reduction over the MLP's outputs rounded up to 64: the surplus columns of g meet zero weights)
            const int kp = num_mlps == 1 ? L.ld_g : (cout_j + 63) / 64 * 64;
            if ((rc = gemm_bf16_nt(g, w, d_proj + (size_t)j * inner_j, rows, inner_j, kp, inner, status, s))) return rc;
        }
        if (tc)
            rc = launch_backward_tc<ARGS, BASIS>(K, args, pts, planes, cin, samples, neighbors, start_ids, radii, (int)m0,
                                                 (int)m1, d_proj, d_feat, d_pts, d_samples, d_param0, d_param1, d_pdf,
                                                 fused_p ? ws + L.p_hi_off : nullptr, fused_p ? ws + L.p_lo_off : nullptr, L.ld_p,
                                                 status, s);
        else
            rc = dispatch_dims<BasisTraits<BASIS>::kOnly3D>(D, [&](auto dim) {
                constexpr int DIM = decltype(dim)::value;
                return launch_backward_pairs<DIM, ARGS, BASIS>(K, args, pts, feats, cin, samples, neighbors, start_ids, radii,
                                                               (int)m0, (int)m1, d_proj, d_feat, d_pts, d_samples, d_param0,
                                                               d_param1, d_pdf, s);
            });
        if (rc) return rc;
        if (fused_p)
            if ((rc = weight_grads())) return rc;
    }
    return publish_status(status, kOriginConvBackward, s);
}

// ---- weight variance -------------------------------------------------------------------------
// The reference's *_compute_weight_variance operators (pcconvs/shared/compute_variance_weights.cu:24-170) return
//     1 / mean_m( s_m^2 * sum_{i, j in seg(m)} (b_i . b_j) (f_i . f_j) ),     s_m = 1 / n_m or 1,
// with a block per sample looping over all n_m^2 pairs of neighbors.  The double sum is the squared Frobenius norm
// of the sample's projected features, || sum_t f_t (x) b_t ||^2 = || P[m] ||^2, so the projection kernels above
// do the work in O(n_m) per sample and a row-norm kernel finishes it.
static __global__ void __launch_bounds__(256)
row_sq_norm_kernel(int rows, int ld_p, const __nv_bfloat16* __restrict__ p_hi, const __nv_bfloat16* __restrict__ p_lo,
                   const int32_t* __restrict__ start_ids, int m_begin, int divide, double* __restrict__ accum) {
    __shared__ double s_part[8];
    const int warp = threadIdx.x >> 5, lane = lane_id();
    double local = 0.0;
    for (int r = blockIdx.x * 8 + warp; r < rows; r += gridDim.x * 8) {
        const size_t row = (size_t)r * ld_p;
        float acc = 0.f;
        for (int c = lane * 2; c < ld_p; c += 64) {
            const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(p_hi + row + c);
            const __nv_bfloat162 l = *reinterpret_cast<const __nv_bfloat162*>(p_lo + row + c);
            const float v0 = __low2float(h) + __low2float(l), v1 = __high2float(h) + __high2float(l);
            acc = fmaf(v0, v0, fmaf(v1, v1, acc));
        }
        acc = warp_sum(acc);
        if (divide) {
            const int m = m_begin + r;
            const int n = __ldg(start_ids + m) - (m > 0 ? __ldg(start_ids + m - 1) : 0);
            acc = n > 0 ? acc / ((float)n * (float)n) : 0.f;
        }
        local += (double)acc;
    }
    if (lane == 0) s_part[warp] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
        for (int i = 0; i < 8; ++i) tot += s_part[i];
        if (tot != 0.0) atomicAdd(accum, tot);
    }
}

static __global__ void finish_weight_var_kernel(const double* __restrict__ accum, long long num_samples, float* __restrict__ out) {
    out[0] = (float)(1.0 / (accum[0] / (double)num_samples));
}

static size_t conv_weight_var_workspace(int64_t num_pts, int64_t num_samples, int cin, int K) {
    const ConvLayout L = conv_layout(num_pts, num_samples, cin, K, 1);
    return L.w_hi_off + 256 + 2 * feature_plane_bytes(num_pts, cin);  // the two P planes, the accumulator, the feature planes
}

template <class ARGS, template <int, int> class BASIS>
static int conv_weight_var(const char* who, int D, int K, const ARGS& args, int64_t num_pts, const float* pts,
                           const float* feats, int cin, int64_t num_samples, const float* samples,
                           const int32_t* neighbors, const int32_t* start_ids, const float* radii, int divide,
                           float* out_variance, void* workspace, size_t workspace_bytes, cudaStream_t s) {
    PCCNN_CHECK_ARG(D >= kMinDims && D <= kMaxDims, "%s: point dimension %d outside [2, 6]", who, D);
    PCCNN_CHECK_ARG(K >= 1 && K <= 64, "%s: basis size %d outside [1, 64]", who, K);
    PCCNN_CHECK_ARG(cin >= 1 && num_samples >= 1 && num_samples < 0x7fffffffLL && num_pts >= 0, "%s: bad sizes", who);
    PCCNN_CHECK_ARG(pts && feats && samples && start_ids && radii && out_variance, "%s: null pointer", who);
    const ConvLayout L = conv_layout(num_pts, num_samples, cin, K, 1);
    const size_t need = conv_weight_var_workspace(num_pts, num_samples, cin, K);
    if (!workspace || workspace_bytes < need) {
        set_error("%s: workspace of %zu bytes, need %zu", who, workspace_bytes, need);
        return PCCNN_ERR_WORKSPACE;
    }
    char* ws = (char*)workspace;
    double* accum = (double*)(ws + L.w_hi_off);
    PCCNN_CUDA(cudaMemsetAsync(accum, 0, 128, s));  // the accumulator and, 64 bytes on, the status word of the kernels
    const bool tc = use_tensor_core_pairs(D, cin);
    const size_t plane = feature_plane_bytes(num_pts, cin);
    const FeaturePlanes planes{(const __nv_bfloat16*)(ws + L.w_hi_off + 256), (const __nv_bfloat16*)(ws + L.w_hi_off + 256 + plane),
                               L.ld_f};
    if (tc)
        if (int rc = split_features(num_pts, cin, feats, ws + L.w_hi_off + 256, ws + L.w_hi_off + 256 + plane, s)) return rc;
    for (int64_t m0 = 0; m0 < num_samples; m0 += L.chunk) {
        const int64_t m1 = (m0 + L.chunk < num_samples) ? m0 + L.chunk : num_samples;
        int rc = PCCNN_OK;
        if (tc)
            rc = launch_project_tc<ARGS, BASIS, true>(K, args, pts, planes, cin, samples, neighbors, start_ids, radii, (int)m0,
                                                      (int)m1, ws + L.p_hi_off, ws + L.p_lo_off, L.ld_p,
                                                      (int*)(ws + L.w_hi_off + 64), s);
        else
            rc = dispatch_dims<BasisTraits<BASIS>::kOnly3D>(D, [&](auto dim) {
                constexpr int DIM = decltype(dim)::value;
                return launch_project<DIM, ARGS, BASIS>(K, args, pts, feats, cin, samples, neighbors, start_ids, radii,
                                                        (int)m0, (int)m1, ws + L.p_hi_off, ws + L.p_lo_off, L.ld_p, s);
            });
        if (rc) return rc;
        row_sq_norm_kernel<<<grid_for((m1 - m0) * 32, 256, 8), 256, 0, s>>>(
            (int)(m1 - m0), L.ld_p, (const __nv_bfloat16*)(ws + L.p_hi_off), (const __nv_bfloat16*)(ws + L.p_lo_off),
            start_ids, (int)m0, divide, accum);
        PCCNN_LAUNCH_CHECK();
    }
    finish_weight_var_kernel<<<1, 1, 0, s>>>(accum, (long long)num_samples, out_variance);
    PCCNN_LAUNCH_CHECK();
    return publish_status((const int*)(ws + L.w_hi_off + 64), kOriginWeightVar, s);
}

}  // namespace pccnn
