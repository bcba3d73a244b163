// Gaussian kernel density estimate over CSR neighbor lists and its point gradients.
//
// Restates pccnn_lib_ops/compute_pdf/compute_pdf.cu:24-149 of phermosilla/pccnn_lib:
//   pdf_i = sum_j  prod_d(ibw_d) * (2*3.1415)^(-md/2) * expf(-0.5 * |(p_j - p_i) * ibw|^2)
// (the constant really is 3.1415, and the reference evaluates the scale in double).
//
// Design: the reference walks a segment with one thread; here one warp owns a point, its
// lanes stream the int2 neighbor rows with coalesced 8-byte loads (the only HBM stream that
// matters: 8 B per pair), gather the neighbor coordinates through L2 and reduce with
// shuffles.  The per-pair scale is hoisted out of the loop.  The gradient kernel reduces
// the "own point" side in the warp and uses one fire-and-forget float reduction per
// coordinate for the neighbor side.
#include "common.cuh"

namespace pccnn {

constexpr int kPdfWarps = 8;

template <int D>
__device__ __forceinline__ float pdf_scale(const float (&ibw)[D], int manifold_dims) {
    float prod = 1.0f;
#pragma unroll
    for (int d = 0; d < D; ++d) prod *= ibw[d];
    const double c = 1.0 / pow(2.0 * 3.1415, (double)manifold_dims / 2.0);
    return (float)((double)prod * c);
}

template <int D>
__global__ void __launch_bounds__(kPdfWarps * 32)
pdf_kernel(int manifold_dims, const float* __restrict__ bandwidth, int n, const float* __restrict__ pts,
           const int2* __restrict__ neighbors, const int32_t* __restrict__ start_ids,
           float* __restrict__ out_pdf) {
    float ibw[D];
#pragma unroll
    for (int d = 0; d < D; ++d) ibw[d] = __frcp_rn(__ldg(bandwidth + d));
    const float scale = pdf_scale<D>(ibw, manifold_dims);
    const int lane = lane_id();
    const int warps_total = gridDim.x * kPdfWarps;
    for (int i = blockIdx.x * kPdfWarps + (threadIdx.x >> 5); i < n; i += warps_total) {
        float p[D];
#pragma unroll
        for (int d = 0; d < D; ++d) p[d] = __ldg(pts + (int64_t)i * D + d);
        const int lo = (i > 0) ? __ldg(start_ids + i - 1) : 0;
        const int hi = __ldg(start_ids + i);
        float acc = 0.f;
        auto term = [&](int j) {
            float dot = 0.f;
#pragma unroll
            for (int d = 0; d < D; ++d) {
                const float v = (__ldg(pts + (int64_t)j * D + d) - p[d]) * ibw[d];
                dot = fmaf(v, v, dot);
            }
            return expf(dot * -0.5f);
        };
        // The loop is bound by memory latency, not arithmetic: four row loads per lane are issued
        // before their gathers, and the four gathers before the first exponential.  The order of the
        // sum is unchanged (one accumulator, ascending t).
        int t = lo + lane;
        for (; t + 96 < hi; t += 128) {
            const int j0 = __ldcs(&neighbors[t]).x;  // streamed once: do not keep in cache
            const int j1 = __ldcs(&neighbors[t + 32]).x;
            const int j2 = __ldcs(&neighbors[t + 64]).x;
            const int j3 = __ldcs(&neighbors[t + 96]).x;
            const float e0 = term(j0), e1 = term(j1), e2 = term(j2), e3 = term(j3);
            acc += e0;
            acc += e1;
            acc += e2;
            acc += e3;
        }
        for (; t < hi; t += 32) acc += term(__ldcs(&neighbors[t]).x);
        acc = warp_sum(acc);
        if (lane == 0) out_pdf[i] = acc * scale;
    }
}

// 3-D points padded to 16 bytes: a neighbor then costs one 128-bit gather instead of three 32-bit ones
// (the gathers, not the 8 B/pair list stream, are what the density kernel waits on).
__global__ void pad_points_kernel(int n, const float* __restrict__ pts, float4* __restrict__ out) {
    const int stride = gridDim.x * blockDim.x;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = make_float4(pts[3 * (int64_t)i], pts[3 * (int64_t)i + 1], pts[3 * (int64_t)i + 2], 0.f);
}

// pdf_kernel<3> on the padded copy: same terms, same order of the sum.
__global__ void __launch_bounds__(kPdfWarps * 32)
pdf_kernel_padded(int manifold_dims, const float* __restrict__ bandwidth, int n, const float4* __restrict__ pts4,
                  const int2* __restrict__ neighbors, const int32_t* __restrict__ start_ids,
                  float* __restrict__ out_pdf) {
    float ibw[3];
#pragma unroll
    for (int d = 0; d < 3; ++d) ibw[d] = __frcp_rn(__ldg(bandwidth + d));
    const float scale = pdf_scale<3>(ibw, manifold_dims);
    const int lane = lane_id();
    const int warps_total = gridDim.x * kPdfWarps;
    for (int i = blockIdx.x * kPdfWarps + (threadIdx.x >> 5); i < n; i += warps_total) {
        const float4 p = __ldg(pts4 + i);
        const int lo = (i > 0) ? __ldg(start_ids + i - 1) : 0;
        const int hi = __ldg(start_ids + i);
        float acc = 0.f;
        auto term = [&](int j) {
            const float4 q = __ldg(pts4 + j);
            const float vx = (q.x - p.x) * ibw[0], vy = (q.y - p.y) * ibw[1], vz = (q.z - p.z) * ibw[2];
            return expf(fmaf(vz, vz, fmaf(vy, vy, fmaf(vx, vx, 0.f))) * -0.5f);
        };
        // eight row loads per lane in flight where the row is long enough (4 % over four), then four, then one
        int t = lo + lane;
        for (; t + 224 < hi; t += 256) {
            int j[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) j[u] = __ldcs(&neighbors[t + 32 * u]).x;
            float e[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) e[u] = term(j[u]);
#pragma unroll
            for (int u = 0; u < 8; ++u) acc += e[u];
        }
        for (; t + 96 < hi; t += 128) {
            const int j0 = __ldcs(&neighbors[t]).x;
            const int j1 = __ldcs(&neighbors[t + 32]).x;
            const int j2 = __ldcs(&neighbors[t + 64]).x;
            const int j3 = __ldcs(&neighbors[t + 96]).x;
            const float e0 = term(j0), e1 = term(j1), e2 = term(j2), e3 = term(j3);
            acc += e0;
            acc += e1;
            acc += e2;
            acc += e3;
        }
        for (; t < hi; t += 32) acc += term(__ldcs(&neighbors[t]).x);
        acc = warp_sum(acc);
        if (lane == 0) out_pdf[i] = acc * scale;
    }
}

template <int D>
__global__ void __launch_bounds__(kPdfWarps * 32)
pdf_grads_kernel(int manifold_dims, const float* __restrict__ bandwidth, int n, const float* __restrict__ pts,
                 const int2* __restrict__ neighbors, const int32_t* __restrict__ start_ids,
                 const float* __restrict__ in_grads, float* __restrict__ out_grads) {
    float ibw[D];
#pragma unroll
    for (int d = 0; d < D; ++d) ibw[d] = __frcp_rn(__ldg(bandwidth + d));
    const float scale = pdf_scale<D>(ibw, manifold_dims);
    const int lane = lane_id();
    const int warps_total = gridDim.x * kPdfWarps;
    for (int i = blockIdx.x * kPdfWarps + (threadIdx.x >> 5); i < n; i += warps_total) {
        float p[D], own[D];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            p[d] = __ldg(pts + (int64_t)i * D + d);
            own[d] = 0.f;
        }
        const int lo = (i > 0) ? __ldg(start_ids + i - 1) : 0;
        const int hi = __ldg(start_ids + i);
        const float gs = __ldg(in_grads + i) * scale;
        for (int t = lo + lane; t < hi; t += 32) {
            const int j = __ldcs(&neighbors[t]).x;
            float v[D], dot = 0.f;
#pragma unroll
            for (int d = 0; d < D; ++d) {
                v[d] = (__ldg(pts + (int64_t)j * D + d) - p[d]) * ibw[d];
                dot = fmaf(v[d], v[d], dot);
            }
            const float w = expf(dot * -0.5f) * gs;
#pragma unroll
            for (int d = 0; d < D; ++d) {
                const float gd = v[d] * ibw[d] * w;
                own[d] += gd;
                if (j != i) atomicAdd(out_grads + (int64_t)j * D + d, -gd);  // compiles to RED.ADD.F32
            }
        }
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const float total = warp_sum(own[d]);
            if (lane == 0 && total != 0.f) atomicAdd(out_grads + (int64_t)i * D + d, total);
        }
    }
}

// Gradient of the density for a list that is the FULL self-neighborhood of the points (every pair (i, j) sits in the
// row of i and in the row of j, which is what the search returns for samples = points with no cap on the count).
// Then the term that sample m's density contributes to point i is the mirror image of a pair in i's own row, and
//     grad_i = scale * sum_{j in N(i)} (g_i + g_j) w_ij (x_j - x_i) / bw^2 ,
// one pass over the row of i with one more gathered value per pair (g_j) and no reduction into other rows at all
// (the general kernel above makes three float reductions per pair into random rows).  The 3-D form gathers
// (x, y, z, g) as one 128-bit load from a padded copy.
template <int D>
__global__ void __launch_bounds__(kPdfWarps * 32)
pdf_grads_symmetric_kernel(int manifold_dims, const float* __restrict__ bandwidth, int n, const float* __restrict__ pts,
                           const int2* __restrict__ neighbors, const int32_t* __restrict__ start_ids,
                           const float* __restrict__ in_grads, float* __restrict__ out_grads) {
    float ibw[D];
#pragma unroll
    for (int d = 0; d < D; ++d) ibw[d] = __frcp_rn(__ldg(bandwidth + d));
    const float scale = pdf_scale<D>(ibw, manifold_dims);
    const int lane = lane_id();
    const int warps_total = gridDim.x * kPdfWarps;
    for (int i = blockIdx.x * kPdfWarps + (threadIdx.x >> 5); i < n; i += warps_total) {
        float p[D], acc[D];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            p[d] = __ldg(pts + (int64_t)i * D + d);
            acc[d] = 0.f;
        }
        const int lo = (i > 0) ? __ldg(start_ids + i - 1) : 0;
        const int hi = __ldg(start_ids + i);
        const float gi = __ldg(in_grads + i);
        for (int t = lo + lane; t < hi; t += 32) {
            const int j = __ldcs(&neighbors[t]).x;
            float v[D], dot = 0.f;
#pragma unroll
            for (int d = 0; d < D; ++d) {
                v[d] = (__ldg(pts + (int64_t)j * D + d) - p[d]) * ibw[d];
                dot = fmaf(v[d], v[d], dot);
            }
            const float w = expf(dot * -0.5f) * (gi + __ldg(in_grads + j));  // j == i: v is zero
#pragma unroll
            for (int d = 0; d < D; ++d) acc[d] = fmaf(v[d] * ibw[d], w, acc[d]);
        }
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const float total = warp_sum(acc[d]);
            if (lane == 0) out_grads[(int64_t)i * D + d] = total * scale;
        }
    }
}

__global__ void pad_points_grads_kernel(int n, const float* __restrict__ pts, const float* __restrict__ in_grads,
                                        float4* __restrict__ out) {
    const int stride = gridDim.x * blockDim.x;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = make_float4(pts[3 * (int64_t)i], pts[3 * (int64_t)i + 1], pts[3 * (int64_t)i + 2], in_grads[i]);
}

__global__ void __launch_bounds__(kPdfWarps * 32)
pdf_grads_symmetric_padded(int manifold_dims, const float* __restrict__ bandwidth, int n, const float4* __restrict__ pg,
                           const int2* __restrict__ neighbors, const int32_t* __restrict__ start_ids,
                           float* __restrict__ out_grads) {
    float ibw[3];
#pragma unroll
    for (int d = 0; d < 3; ++d) ibw[d] = __frcp_rn(__ldg(bandwidth + d));
    const float scale = pdf_scale<3>(ibw, manifold_dims);
    const int lane = lane_id();
    const int warps_total = gridDim.x * kPdfWarps;
    for (int i = blockIdx.x * kPdfWarps + (threadIdx.x >> 5); i < n; i += warps_total) {
        const float4 p = __ldg(pg + i);
        const int lo = (i > 0) ? __ldg(start_ids + i - 1) : 0;
        const int hi = __ldg(start_ids + i);
        float ax = 0.f, ay = 0.f, az = 0.f;
        auto term = [&](int j) {
            const float4 q = __ldg(pg + j);
            const float vx = (q.x - p.x) * ibw[0], vy = (q.y - p.y) * ibw[1], vz = (q.z - p.z) * ibw[2];
            const float w = expf(fmaf(vz, vz, fmaf(vy, vy, fmaf(vx, vx, 0.f))) * -0.5f) * (p.w + q.w);
            ax = fmaf(vx * ibw[0], w, ax);
            ay = fmaf(vy * ibw[1], w, ay);
            az = fmaf(vz * ibw[2], w, az);
        };
        // as in the density kernel: four row loads per lane in flight before their gathers
        int t = lo + lane;
        for (; t + 96 < hi; t += 128) {
            const int j0 = __ldcs(&neighbors[t]).x;
            const int j1 = __ldcs(&neighbors[t + 32]).x;
            const int j2 = __ldcs(&neighbors[t + 64]).x;
            const int j3 = __ldcs(&neighbors[t + 96]).x;
            term(j0);
            term(j1);
            term(j2);
            term(j3);
        }
        for (; t < hi; t += 32) term(__ldcs(&neighbors[t]).x);
        ax = warp_sum(ax);
        ay = warp_sum(ay);
        az = warp_sum(az);
        if (lane == 0) {
            out_grads[3 * (int64_t)i] = ax * scale;
            out_grads[3 * (int64_t)i + 1] = ay * scale;
            out_grads[3 * (int64_t)i + 2] = az * scale;
        }
    }
}

}  // namespace pccnn

using namespace pccnn;

extern "C" {

size_t pccnn_compute_pdf_workspace_bytes(int D, int64_t n) { return (D == 3 && n > 0) ? (size_t)n * 16 : 0; }

int pccnn_compute_pdf(int D, int manifold_dims, const float* bandwidth, int64_t n, const float* pts,
                      const int32_t* neighbors, const int32_t* start_ids, float* out_pdf, void* workspace,
                      size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(n >= 0 && n < 0x7fffffffLL, "compute_pdf: %lld points outside [0, 2^31)", (long long)n);
    if (n == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(bandwidth && pts && start_ids && out_pdf, "compute_pdf: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned grid = grid_for(n * 32, kPdfWarps * 32, 8);
    if (D == 3 && workspace && workspace_bytes >= (size_t)n * 16 && reinterpret_cast<uintptr_t>(workspace) % 16 == 0) {
        // optional scratch given: gather from a 16-byte padded copy of the points
        float4* padded = (float4*)workspace;
        pad_points_kernel<<<grid_for(n, 256, 8), 256, 0, s>>>((int)n, pts, padded);
        PCCNN_LAUNCH_CHECK();
        pdf_kernel_padded<<<resident_grid(pdf_kernel_padded, n * 32, kPdfWarps * 32), kPdfWarps * 32, 0, s>>>(
            manifold_dims, bandwidth, (int)n, padded, (const int2*)neighbors, start_ids, out_pdf);
        PCCNN_LAUNCH_CHECK();
        return PCCNN_OK;
    }
    PCCNN_DISPATCH_DIM(D, (pdf_kernel<DIM><<<grid, kPdfWarps * 32, 0, s>>>(
                              manifold_dims, bandwidth, (int)n, pts, (const int2*)neighbors, start_ids, out_pdf)));
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

int pccnn_compute_pdf_grads(int D, int manifold_dims, const float* bandwidth, int64_t n, const float* pts,
                            const int32_t* neighbors, const int32_t* start_ids, const float* in_grads,
                            float* out_pt_grads, void* stream) {
    PCCNN_CHECK_ARG(n >= 0 && n < 0x7fffffffLL, "compute_pdf_grads: %lld points outside [0, 2^31)", (long long)n);
    PCCNN_CHECK_ARG(D >= kMinDims && D <= kMaxDims, "compute_pdf_grads: point dimension %d outside [2, 6]", D);
    if (n == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(bandwidth && pts && start_ids && in_grads && out_pt_grads, "compute_pdf_grads: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    PCCNN_CUDA(cudaMemsetAsync(out_pt_grads, 0, (size_t)n * D * sizeof(float), s));
    PCCNN_DISPATCH_DIM(D, (pdf_grads_kernel<DIM><<<resident_grid(pdf_grads_kernel<DIM>, n * 32, kPdfWarps * 32),
                                                   kPdfWarps * 32, 0, s>>>(
                              manifold_dims, bandwidth, (int)n, pts, (const int2*)neighbors, start_ids, in_grads,
                              out_pt_grads)));
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

int pccnn_compute_pdf_grads_symmetric(int D, int manifold_dims, const float* bandwidth, int64_t n, const float* pts,
                                      const int32_t* neighbors, const int32_t* start_ids, const float* in_grads,
                                      float* out_pt_grads, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(n >= 0 && n < 0x7fffffffLL, "compute_pdf_grads_symmetric: %lld points outside [0, 2^31)", (long long)n);
    if (n == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(bandwidth && pts && start_ids && in_grads && out_pt_grads, "compute_pdf_grads_symmetric: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    if (D == 3 && workspace && workspace_bytes >= (size_t)n * 16 && reinterpret_cast<uintptr_t>(workspace) % 16 == 0) {
        float4* padded = (float4*)workspace;
        pad_points_grads_kernel<<<grid_for(n, 256, 8), 256, 0, s>>>((int)n, pts, in_grads, padded);
        PCCNN_LAUNCH_CHECK();
        pdf_grads_symmetric_padded<<<resident_grid(pdf_grads_symmetric_padded, n * 32, kPdfWarps * 32), kPdfWarps * 32, 0,
                                     s>>>(manifold_dims, bandwidth, (int)n, padded, (const int2*)neighbors, start_ids,
                                          out_pt_grads);
        PCCNN_LAUNCH_CHECK();
        return PCCNN_OK;
    }
    PCCNN_DISPATCH_DIM(D, (pdf_grads_symmetric_kernel<DIM><<<resident_grid(pdf_grads_symmetric_kernel<DIM>, n * 32,
                                                                          kPdfWarps * 32),
                                                             kPdfWarps * 32, 0, s>>>(
                              manifold_dims, bandwidth, (int)n, pts, (const int2*)neighbors, start_ids, in_grads,
                              out_pt_grads)));
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

}  // extern "C"
