// SPHConv and PointConv: a one-hot spherical-bin basis, and a basis supplied by the caller.
//
// Restates pccnn_lib_ops/pcconvs/sphconv.cu:32-146 (basis shared/spherical_basis.cu:24-168) and
// pointconv.cu:32-139 of phermosilla/pccnn_lib on the projection / contraction templates of conv_impl.cuh.
//   SPHConv:   b[t, k] = [k == bin(d_t)], k = 0 for |d_t| < 1e-4, else 1 + (radial bin * A + azimuth bin) * P + polar bin;
//              out[m] = (P[m] W) / (n_m + 1e-6).  The division is folded into the basis (b / (n_m + 1e-6)): the
//              operator is linear in b, so output, weight and feature gradients are the reference's.
//   PointConv: the [T, K] basis is an input (the layer passes the affine projection of pointconv_basis through its
//              own batch norm / ReLU / density MLP in Python first); the basis gradient is an output.
#include "conv_impl.cuh"

namespace pccnn {

struct SphArgs {
    const float* radial_bins;   // [R] upper bin edges, ascending
    const float* azimuth_bins;  // [A]
    const float* polar_bins;    // [P]
    int nr, na, np;
    const int32_t* start_ids;   // [M] inclusive ends: the neighbor count scales the basis
};

template <int D, int KP>
struct SphBasis {
    static constexpr bool kUsesOffset = true;
    static constexpr int kParamFloats = 64;  // up to 64 bin edges in total
    static constexpr int kGradFloats = 1;
    __device__ static void load_params(float* sp, const SphArgs& a, int /*K*/) {
        for (int i = threadIdx.x; i < 64; i += blockDim.x) {
            float v = 0.f;
            if (i < a.nr) v = __ldg(a.radial_bins + i);
            else if (i < a.nr + a.na) v = __ldg(a.azimuth_bins + i - a.nr);
            else if (i < a.nr + a.na + a.np) v = __ldg(a.polar_bins + i - a.nr - a.na);
            sp[i] = v;
        }
    }
    __device__ static int first_bin(const float* edges, int n, float v) {
        for (int i = 0; i < n; ++i)
            if (v <= edges[i]) return i;
        return n - 1;
    }
    __device__ static void eval(const float* sp, const SphArgs& a, int K, const float (&d)[D], int /*n0*/, int /*t*/, int m,
                                float (&b)[KP]) {
        // spherical_basis.cu:141-158: distance, azimuth atan(y / (x + 1e-6)), polar acos(clamp(z / (dist + 1e-6)))
        const float x = d[0], y = d[D > 1 ? 1 : 0], z = d[D > 2 ? 2 : 0];
        const float dist = sqrtf(__fadd_rn(__fadd_rn(__fmul_rn(x, x), __fmul_rn(y, y)), __fmul_rn(z, z)));
        const float az = atanf(__fdiv_rn(y, __fadd_rn(x, 1e-6f)));
        const float pol = acosf(fminf(fmaxf(__fdiv_rn(z, __fadd_rn(dist, 1e-6f)), -0.99999f), 0.99999f));
        int id = 0;
        if (!(dist < 1e-4f)) {
            const int r = first_bin(sp, a.nr, dist), az_id = first_bin(sp + a.nr, a.na, az);
            const int p = first_bin(sp + a.nr + a.na, a.np, pol);
            id = r * a.na * a.np + az_id * a.np + p + 1;
        }
        const int n = __ldg(a.start_ids + m) - (m > 0 ? __ldg(a.start_ids + m - 1) : 0);
        const float scale = 1.0f / ((float)n + 1e-6f);
#pragma unroll
        for (int k = 0; k < KP; ++k) b[k] = (k == id && k < K) ? scale : 0.f;
    }
    // The reference returns weight and feature gradients only (sphconv.cu:106): the bins are not differentiable.
    __device__ static void grad(const float*, const SphArgs&, int, const float (&)[D], int, int, int, bool, const float*,
                                float (&)[D], float*, float&) {}
    __device__ static void grad_local(const float*, const SphArgs&, int, const float (&)[D], int, int, int, bool,
                                      const float*, float (&)[D], float (&)[kGradFloats], float&) {}
    __device__ static void flush(const float*, int, float*, float*) {}
};
template <>
struct BasisTraits<SphBasis> {
    static constexpr bool kOnly3D = true;
};

struct TableArgs {
    const float* basis;  // [T, K]
    float* d_basis;      // [T, K], backward only
};

template <int D, int KP>
struct TableBasis {
    static constexpr bool kUsesOffset = false;  // points, samples and radii are never read
    static constexpr int kParamFloats = 1;
    static constexpr int kGradFloats = 1;
    __device__ static void load_params(float*, const TableArgs&, int) {}
    __device__ static void eval(const float*, const TableArgs& a, int K, const float (&)[D], int /*n0*/, int t, int /*m*/,
                                float (&b)[KP]) {
        const float* row = a.basis + (size_t)t * K;
#pragma unroll
        for (int k = 0; k < KP; ++k) b[k] = (k < K) ? __ldg(row + k) : 0.f;
    }
    __device__ static void grad(const float*, const TableArgs& a, int K, const float (&)[D], int, int t, int, bool active,
                                const float* db, float (&)[D], float*, float&) {
        if (active)
            for (int k = 0; k < K; ++k) a.d_basis[(size_t)t * K + k] = db[k];
    }
    __device__ static void grad_local(const float* sp, const TableArgs& a, int K, const float (&d)[D], int n0, int t, int m,
                                      bool active, const float* db, float (&d_off)[D], float (&)[kGradFloats], float& dp) {
        grad(sp, a, K, d, n0, t, m, active, db, d_off, nullptr, dp);
    }
    __device__ static void flush(const float*, int, float*, float*) {}
};
template <>
struct BasisTraits<TableBasis> {
    static constexpr bool kOnly3D = true;  // the dimension plays no role: one instantiation
};

// point_conv_basis: [T, K] = ((pts[n0] - samples[n1]) / radii) . axis + bias      (pointconv.cu:32-51)
template <int D>
static __global__ void __launch_bounds__(256)
affine_basis_kernel(int64_t total, int K, const float* __restrict__ pts, const float* __restrict__ samples,
                    const int2* __restrict__ neighbors, const float* __restrict__ radii, const float* __restrict__ axis,
                    const float* __restrict__ bias, float* __restrict__ out) {
    float inv[D];
#pragma unroll
    for (int d = 0; d < D; ++d) inv[d] = __frcp_rn(__ldg(radii + d));
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total * K; i += stride) {
        const int64_t t = i / K;
        const int k = (int)(i - t * K);
        const int2 row = __ldg(neighbors + t);
        float acc = 0.f;
#pragma unroll
        for (int d = 0; d < D; ++d)
            acc = fmaf((__ldg(pts + (int64_t)row.x * D + d) - __ldg(samples + (int64_t)row.y * D + d)) * inv[d],
                       __ldg(axis + d * K + k), acc);
        out[i] = acc + __ldg(bias + k);
    }
}

// Gradients of point_conv_basis (pointconv.cu:54-86): a warp takes 32 pairs at a time.
template <int D>
static __global__ void __launch_bounds__(256)
affine_basis_grads_kernel(int64_t total, int K, const float* __restrict__ pts, const float* __restrict__ samples,
                          const int2* __restrict__ neighbors, const float* __restrict__ radii,
                          const float* __restrict__ axis, const float* __restrict__ grads, float* __restrict__ d_pts,
                          float* __restrict__ d_samples, float* __restrict__ d_axis, float* __restrict__ d_bias) {
    extern __shared__ float s_acc[];  // [(D + 1) * K]: axis gradient rows, then the bias gradient
    for (int i = threadIdx.x; i < (D + 1) * K; i += blockDim.x) s_acc[i] = 0.f;
    __syncthreads();
    float inv[D];
#pragma unroll
    for (int d = 0; d < D; ++d) inv[d] = __frcp_rn(__ldg(radii + d));
    const int lane = lane_id();
    const int64_t warp_global = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t t0 = warp_global * 32; t0 < total; t0 += warps * 32) {
        const int64_t t = t0 + lane;
        const bool active = t < total;
        int2 row = make_int2(0, 0);
        float diff[D], d_off[D];
#pragma unroll
        for (int d = 0; d < D; ++d) diff[d] = d_off[d] = 0.f;
        if (active) {
            row = __ldg(neighbors + t);
#pragma unroll
            for (int d = 0; d < D; ++d)
                diff[d] = (__ldg(pts + (int64_t)row.x * D + d) - __ldg(samples + (int64_t)row.y * D + d)) * inv[d];
        }
        for (int k = 0; k < K; ++k) {
            const float g = active ? __ldg(grads + t * K + k) : 0.f;
            const float tot = warp_sum(g);
            if (lane == 0 && tot != 0.f) atomicAdd(s_acc + D * K + k, tot);
#pragma unroll
            for (int d = 0; d < D; ++d) {
                d_off[d] = fmaf(g, __ldg(axis + d * K + k), d_off[d]);
                const float ta = warp_sum(diff[d] * g);
                if (lane == 0 && ta != 0.f) atomicAdd(s_acc + d * K + k, ta);
            }
        }
        if (active) {
#pragma unroll
            for (int d = 0; d < D; ++d) {
                const float gx = d_off[d] * inv[d];
                if (gx != 0.f) {
                    atomicAdd(d_pts + (int64_t)row.x * D + d, gx);
                    atomicAdd(d_samples + (int64_t)row.y * D + d, -gx);
                }
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < (D + 1) * K; i += blockDim.x) {
        const float v = s_acc[i];
        if (v != 0.f) atomicAdd(i < D * K ? d_axis + i : d_bias + (i - D * K), v);
    }
}

static int check_bins(const char* who, const float* r, const float* a, const float* p, int nr, int na, int np) {
    PCCNN_CHECK_ARG(r && a && p && nr >= 1 && na >= 1 && np >= 1, "%s: bin edges missing", who);
    PCCNN_CHECK_ARG(nr + na + np <= 64 && nr * na * np + 1 <= 64,
                    "%s: at most 64 bin edges and 64 basis functions (got %d x %d x %d bins)", who, nr, na, np);
    return PCCNN_OK;
}

}  // namespace pccnn

using namespace pccnn;

extern "C" {

int pccnn_sph_conv(int D, int64_t num_pts, const float* pts, const float* feats, int cin, int64_t num_samples,
                   const float* samples, const int32_t* neighbors, const int32_t* start_ids, const float* radii,
                   const float* radial_bins, int num_radial, const float* azimuth_bins, int num_azimuth,
                   const float* polar_bins, int num_polar, const float* weights, int cout, float* out, void* workspace,
                   size_t workspace_bytes, void* stream) {
    if (int rc = check_bins("sph_conv", radial_bins, azimuth_bins, polar_bins, num_radial, num_azimuth, num_polar)) return rc;
    SphArgs args{radial_bins, azimuth_bins, polar_bins, num_radial, num_azimuth, num_polar, start_ids};
    return conv_forward<SphArgs, SphBasis>("sph_conv", D, num_radial * num_azimuth * num_polar + 1, args, num_pts, pts,
                                           feats, cin, num_samples, samples, neighbors, start_ids, radii, 1, weights, cout,
                                           out, workspace, workspace_bytes, (cudaStream_t)stream);
}

int pccnn_sph_conv_grads(int D, int64_t num_pts, const float* pts, const float* feats, int cin, int64_t num_samples,
                         const float* samples, const int32_t* neighbors, const int32_t* start_ids, const float* radii,
                         const float* radial_bins, int num_radial, const float* azimuth_bins, int num_azimuth,
                         const float* polar_bins, int num_polar, const float* weights, int cout, const float* in_grads,
                         float* out_weight_grads, float* out_feat_grads, void* workspace, size_t workspace_bytes,
                         void* stream) {
    if (int rc = check_bins("sph_conv_grads", radial_bins, azimuth_bins, polar_bins, num_radial, num_azimuth, num_polar))
        return rc;
    SphArgs args{radial_bins, azimuth_bins, polar_bins, num_radial, num_azimuth, num_polar, start_ids};
    return conv_backward<SphArgs, SphBasis>("sph_conv_grads", D, num_radial * num_azimuth * num_polar + 1, args, num_pts, pts,
                                            feats, cin, num_samples, samples, neighbors, start_ids, radii, 1, weights, cout,
                                            in_grads, out_weight_grads, out_feat_grads, nullptr, 0, nullptr, 0, nullptr,
                                            nullptr, nullptr, workspace, workspace_bytes, (cudaStream_t)stream);
}

int pccnn_sph_conv_weight_var(int D, int64_t num_pts, const float* pts, const float* feats, int cin, int64_t num_samples,
                              const float* samples, const int32_t* neighbors, const int32_t* start_ids, const float* radii,
                              const float* radial_bins, int num_radial, const float* azimuth_bins, int num_azimuth,
                              const float* polar_bins, int num_polar, float* out_variance, void* workspace,
                              size_t workspace_bytes, void* stream) {
    if (int rc = check_bins("sph_conv_weight_var", radial_bins, azimuth_bins, polar_bins, num_radial, num_azimuth, num_polar))
        return rc;
    // The reference evaluates the variance on the one-hot basis and divides by the neighbor count inside
    // compute_variance_weights (pDivideNumNeighs = true, sphconv.cu:145); here the basis already carries
    // 1 / (n + 1e-6), which is that division up to the 1e-6.
    SphArgs args{radial_bins, azimuth_bins, polar_bins, num_radial, num_azimuth, num_polar, start_ids};
    return conv_weight_var<SphArgs, SphBasis>("sph_conv_weight_var", D, num_radial * num_azimuth * num_polar + 1, args,
                                              num_pts, pts, feats, cin, num_samples, samples, neighbors, start_ids, radii, 0,
                                              out_variance, workspace, workspace_bytes, (cudaStream_t)stream);
}

int pccnn_point_conv_basis(int D, int64_t num_pairs, const float* pts, const float* radii, const float* samples,
                           const int32_t* neighbors, const float* axis, const float* bias, int hidden, float* out_basis,
                           void* stream) {
    PCCNN_CHECK_ARG(D >= kMinDims && D <= kMaxDims && hidden >= 1 && num_pairs >= 0, "point_conv_basis: bad sizes");
    if (num_pairs == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(pts && radii && samples && neighbors && axis && bias && out_basis, "point_conv_basis: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    PCCNN_DISPATCH_DIM(D, (affine_basis_kernel<DIM><<<grid_for(num_pairs * hidden, 256, 8), 256, 0, s>>>(
                              num_pairs, hidden, pts, samples, (const int2*)neighbors, radii, axis, bias, out_basis)));
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

int pccnn_point_conv_basis_grads(int D, int64_t num_pts, int64_t num_samples, int64_t num_pairs, const float* pts,
                                 const float* radii, const float* samples, const int32_t* neighbors, const float* axis,
                                 int hidden, const float* in_grads, float* out_pt_grads, float* out_sample_grads,
                                 float* out_axis_grads, float* out_bias_grads, void* stream) {
    PCCNN_CHECK_ARG(D >= kMinDims && D <= kMaxDims && hidden >= 1 && hidden <= 1024 && num_pairs >= 0,
                    "point_conv_basis_grads: bad sizes");
    PCCNN_CHECK_ARG(out_pt_grads && out_sample_grads && out_axis_grads && out_bias_grads, "point_conv_basis_grads: null output");
    cudaStream_t s = (cudaStream_t)stream;
    PCCNN_CUDA(cudaMemsetAsync(out_pt_grads, 0, (size_t)num_pts * D * 4, s));
    PCCNN_CUDA(cudaMemsetAsync(out_sample_grads, 0, (size_t)num_samples * D * 4, s));
    PCCNN_CUDA(cudaMemsetAsync(out_axis_grads, 0, (size_t)D * hidden * 4, s));
    PCCNN_CUDA(cudaMemsetAsync(out_bias_grads, 0, (size_t)hidden * 4, s));
    if (num_pairs == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(pts && radii && samples && neighbors && axis && in_grads, "point_conv_basis_grads: null pointer");
    PCCNN_DISPATCH_DIM(D, (affine_basis_grads_kernel<DIM><<<grid_for(num_pairs, 256, 4), 256, (DIM + 1) * hidden * 4, s>>>(
                              num_pairs, hidden, pts, samples, (const int2*)neighbors, radii, axis, in_grads, out_pt_grads,
                              out_sample_grads, out_axis_grads, out_bias_grads)));
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

int pccnn_point_conv(int64_t num_pts, const float* basis, int hidden, const float* feats, int cin, int64_t num_samples,
                     const int32_t* neighbors, const int32_t* start_ids, const float* weights, int cout, float* out,
                     void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(basis || num_samples == 0, "point_conv: null basis");
    TableArgs args{basis, nullptr};
    // points, samples and radii are not part of this operator; the kernels never read them for this basis
    const float* unused = feats;
    return conv_forward<TableArgs, TableBasis>("point_conv", 3, hidden, args, num_pts, unused, feats, cin, num_samples,
                                               unused, neighbors, start_ids, unused, 1, weights, cout, out, workspace,
                                               workspace_bytes, (cudaStream_t)stream);
}

int pccnn_point_conv_grads(int64_t num_pts, const float* basis, int hidden, const float* feats, int cin,
                           int64_t num_samples, int64_t num_pairs, const int32_t* neighbors, const int32_t* start_ids,
                           const float* weights, int cout, const float* in_grads, float* out_weight_grads,
                           float* out_feat_grads, float* out_basis_grads, void* workspace, size_t workspace_bytes,
                           void* stream) {
    PCCNN_CHECK_ARG((basis && out_basis_grads) || num_pairs == 0, "point_conv_grads: null basis");
    if (out_basis_grads && num_pairs > 0)
        PCCNN_CUDA(cudaMemsetAsync(out_basis_grads, 0, (size_t)num_pairs * hidden * 4, (cudaStream_t)stream));
    TableArgs args{basis, out_basis_grads};
    const float* unused = feats;
    return conv_backward<TableArgs, TableBasis>("point_conv_grads", 3, hidden, args, num_pts, unused, feats, cin,
                                                num_samples, unused, neighbors, start_ids, unused, 1, weights, cout, in_grads,
                                                out_weight_grads, out_feat_grads, nullptr, 0, nullptr, 0, nullptr, nullptr,
                                                nullptr, workspace, workspace_bytes, (cudaStream_t)stream);
}

int pccnn_point_conv_weight_var(int64_t num_pts, const float* basis, int hidden, const float* feats, int cin,
                                int64_t num_samples, const int32_t* neighbors, const int32_t* start_ids,
                                float* out_variance, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(basis, "point_conv_weight_var: null basis");
    TableArgs args{basis, nullptr};
    const float* unused = feats;
    return conv_weight_var<TableArgs, TableBasis>("point_conv_weight_var", 3, hidden, args, num_pts, unused, feats, cin,
                                                  num_samples, unused, neighbors, start_ids, unused, 0, out_variance,
                                                  workspace, workspace_bytes, (cudaStream_t)stream);
}

}  // extern "C"
