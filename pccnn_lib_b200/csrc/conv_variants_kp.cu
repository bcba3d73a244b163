// KPConvN and PCCNN: kernel-point convolutions whose basis is divided by the neighbor's density.
//
// Restates pccnn_lib_ops/pcconvs/kpconvn.cu:32-155 and pccnn.cu:32-165 of phermosilla/pccnn_lib:
//     KPConvN:  b[t, k] = clamp(1 - |kp_k - d_t| / sigma, 0, 1) / pdf[n0(t)]        (shared/kernel_pts_basis.cu:23-70)
//     PCCNN:    b[t, k] = exp(-|kp_k - d_t|^2 / (2 sigma^2)) / pdf[n0(t)]           (shared/kernel_pts_basis.cu:72-111)
// followed by the projection and contraction shared with KPConv (conv_impl.cuh).
#include "conv_impl.cuh"

namespace pccnn {

struct KPDensityArgs {
    const float* kernel_pts;  // [K, D]
    float inv_sigma;          // KPConvN: 1 / sigma;  PCCNN: 1 / sigma^2
    const float* pdf;         // [N]
};

template <int D, int KP>
struct KPNBasis {
    static constexpr bool kUsesOffset = true;
    static constexpr int kParamFloats = KP * D;
    static constexpr int kGradFloats = KP * D;
    __device__ static void load_params(float* sp, const KPDensityArgs& a, int K) {
        for (int i = threadIdx.x; i < KP * D; i += blockDim.x) sp[i] = (i < K * D) ? __ldg(a.kernel_pts + i) : 0.f;
    }
    __device__ static void eval(const float* sp, const KPDensityArgs& a, int K, const float (&d)[D], int n0, int, int,
                                float (&b)[KP]) {
        const float inv_pdf = 1.0f / __ldg(a.pdf + n0);
#pragma unroll
        for (int k = 0; k < KP; ++k) {
            float acc = 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) {
                const float v = sp[k * D + x] - d[x];
                acc = fmaf(v, v, acc);
            }
            const float val = 1.0f - sqrtf(fmaxf(acc, 0.f)) * a.inv_sigma;
            b[k] = (k < K) ? fminf(fmaxf(val, 0.f), 1.f) * inv_pdf : 0.f;
        }
    }
    // kpconvn.cu:118-127: the basis gradient is divided by the density, then kernel_pts_basis_grads; the
    // reference returns no density gradient for this operator.
    __device__ static void grad(const float* sp, const KPDensityArgs& a, int K, const float (&d)[D], int n0, int, int,
                                bool active, const float* db, float (&d_off)[D], float* s_grad, float&) {
        const int lane = lane_id();
        const float inv_pdf = active ? 1.0f / __ldg(a.pdf + n0) : 0.f;
        for (int k = 0; k < K; ++k) {
            float v[D], acc = 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) {
                v[x] = sp[k * D + x] - d[x];
                acc = fmaf(v[x], v[x], acc);
            }
            const float dist = sqrtf(fmaxf(acc, 0.f));
            float gk = 0.f;
            if (active && 1.0f - dist * a.inv_sigma >= 0.f) gk = -db[k] * inv_pdf * a.inv_sigma / (dist + 1e-6f);
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
    __device__ static void grad_local(const float* sp, const KPDensityArgs& a, int K, const float (&d)[D], int n0, int,
                                      int, bool active, const float* db, float (&d_off)[D], float (&acc_g)[kGradFloats],
                                      float&) {
        const float inv_pdf = active ? 1.0f / __ldg(a.pdf + n0) : 0.f;
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
            if (active && k < K && 1.0f - dist * a.inv_sigma >= 0.f) gk = -db[k] * inv_pdf * a.inv_sigma / (dist + 1e-6f);
#pragma unroll
            for (int x = 0; x < D; ++x) {
                const float t = gk * v[x];
                d_off[x] -= t;
                acc_g[k * D + x] += t;
            }
        }
    }
    __device__ static void flush(const float* s_grad, int K, float* g0, float*) {
        for (int i = threadIdx.x; i < K * D; i += blockDim.x)
            if (s_grad[i] != 0.f) atomicAdd(g0 + i, s_grad[i]);
    }
};

template <int D, int KP>
struct GaussBasis {
    static constexpr bool kUsesOffset = true;
    static constexpr int kParamFloats = KP * D;
    static constexpr int kGradFloats = KP * D;
    __device__ static void load_params(float* sp, const KPDensityArgs& a, int K) {
        for (int i = threadIdx.x; i < KP * D; i += blockDim.x) sp[i] = (i < K * D) ? __ldg(a.kernel_pts + i) : 0.f;
    }
    __device__ static void eval(const float* sp, const KPDensityArgs& a, int K, const float (&d)[D], int n0, int, int,
                                float (&b)[KP]) {
        const float inv_pdf = 1.0f / __ldg(a.pdf + n0);
#pragma unroll
        for (int k = 0; k < KP; ++k) {
            float acc = 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) {
                const float v = sp[k * D + x] - d[x];
                acc = fmaf(v, v, acc);
            }
            b[k] = (k < K) ? expf(-0.5f * acc * a.inv_sigma) * inv_pdf : 0.f;
        }
    }
    // pccnn.cu:119-131 with kernel_pts_basis_gauss_grads: dL/dkp = -g e (kp - d) / sigma^2, dL/dd = +g e (kp - d) /
    // sigma^2 with g = db / pdf, and dL/dpdf = -sum_k e db / pdf^2.
    __device__ static void grad(const float* sp, const KPDensityArgs& a, int K, const float (&d)[D], int n0, int, int,
                                bool active, const float* db, float (&d_off)[D], float* s_grad, float& d_pdf) {
        const int lane = lane_id();
        const float inv_pdf = active ? 1.0f / __ldg(a.pdf + n0) : 0.f;
        for (int k = 0; k < K; ++k) {
            float v[D], acc = 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) {
                v[x] = sp[k * D + x] - d[x];
                acc = fmaf(v[x], v[x], acc);
            }
            const float e = expf(-0.5f * acc * a.inv_sigma);
            const float dbk = active ? db[k] : 0.f;
            d_pdf -= e * dbk * inv_pdf * inv_pdf;
            const float g = dbk * inv_pdf * e * a.inv_sigma;
            if (!__any_sync(kFullMask, g != 0.f)) continue;
#pragma unroll
            for (int x = 0; x < D; ++x) {
                const float t = g * v[x];
                d_off[x] += t;
                const float tot = warp_sum(t);
                if (lane == 0) atomicAdd(s_grad + k * D + x, -tot);
            }
        }
    }
    __device__ static void grad_local(const float* sp, const KPDensityArgs& a, int K, const float (&d)[D], int n0, int,
                                      int, bool active, const float* db, float (&d_off)[D], float (&acc_g)[kGradFloats],
                                      float& d_pdf) {
        const float inv_pdf = active ? 1.0f / __ldg(a.pdf + n0) : 0.f;
#pragma unroll
        for (int k = 0; k < KP; ++k) {
            float v[D], acc = 0.f;
#pragma unroll
            for (int x = 0; x < D; ++x) {
                v[x] = sp[k * D + x] - d[x];
                acc = fmaf(v[x], v[x], acc);
            }
            const float e = expf(-0.5f * acc * a.inv_sigma);
            const float dbk = (active && k < K) ? db[k] : 0.f;
            d_pdf -= e * dbk * inv_pdf * inv_pdf;
            const float g = dbk * inv_pdf * e * a.inv_sigma;
#pragma unroll
            for (int x = 0; x < D; ++x) {
                const float t = g * v[x];
                d_off[x] += t;
                acc_g[k * D + x] -= t;
            }
        }
    }
    __device__ static void flush(const float* s_grad, int K, float* g0, float*) {
        for (int i = threadIdx.x; i < K * D; i += blockDim.x)
            if (s_grad[i] != 0.f) atomicAdd(g0 + i, s_grad[i]);
    }
};

}  // namespace pccnn

using namespace pccnn;

extern "C" {

int pccnn_kp_conv_n(int D, int64_t num_pts, const float* pts, const float* pdf, const float* feats, int cin,
                    int64_t num_samples, const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                    const float* radii, const float* kernel_pts, int num_kernel_pts, float sigma, const float* weights,
                    int cout, float* out, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(kernel_pts && pdf && sigma > 0.f, "kp_conv_n: kernel points or density missing, or sigma <= 0");
    KPDensityArgs args{kernel_pts, 1.0f / sigma, pdf};
    return conv_forward<KPDensityArgs, KPNBasis>("kp_conv_n", D, num_kernel_pts, args, num_pts, pts, feats, cin,
                                                 num_samples, samples, neighbors, start_ids, radii, 1, weights, cout, out,
                                                 workspace, workspace_bytes, (cudaStream_t)stream);
}

int pccnn_kp_conv_n_grads(int D, int64_t num_pts, const float* pts, const float* pdf, const float* feats, int cin,
                          int64_t num_samples, const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                          const float* radii, const float* kernel_pts, int num_kernel_pts, float sigma,
                          const float* weights, int cout, const float* in_grads, float* out_weight_grads,
                          float* out_feat_grads, float* out_kernel_pt_grads, float* out_pt_grads, float* out_sample_grads,
                          void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(kernel_pts && pdf && sigma > 0.f, "kp_conv_n_grads: kernel points or density missing, or sigma <= 0");
    PCCNN_CHECK_ARG(out_kernel_pt_grads && out_pt_grads && out_sample_grads, "kp_conv_n_grads: null output");
    KPDensityArgs args{kernel_pts, 1.0f / sigma, pdf};
    return conv_backward<KPDensityArgs, KPNBasis>(
        "kp_conv_n_grads", D, num_kernel_pts, args, num_pts, pts, feats, cin, num_samples, samples, neighbors, start_ids,
        radii, 1, weights, cout, in_grads, out_weight_grads, out_feat_grads, out_kernel_pt_grads,
        (size_t)num_kernel_pts * D, nullptr, 0, nullptr, out_pt_grads, out_sample_grads, workspace, workspace_bytes,
        (cudaStream_t)stream);
}

int pccnn_kp_conv_n_weight_var(int D, int64_t num_pts, const float* pts, const float* pdf, const float* feats, int cin,
                               int64_t num_samples, const float* samples, const int32_t* neighbors,
                               const int32_t* start_ids, const float* radii, const float* kernel_pts, int num_kernel_pts,
                               float sigma, float* out_variance, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(kernel_pts && pdf && sigma > 0.f, "kp_conv_n_weight_var: kernel points or density missing, or sigma <= 0");
    KPDensityArgs args{kernel_pts, 1.0f / sigma, pdf};
    return conv_weight_var<KPDensityArgs, KPNBasis>("kp_conv_n_weight_var", D, num_kernel_pts, args, num_pts, pts, feats,
                                                    cin, num_samples, samples, neighbors, start_ids, radii, 0,
                                                    out_variance, workspace, workspace_bytes, (cudaStream_t)stream);
}

int pccnn_pccnn_conv(int D, int64_t num_pts, const float* pts, const float* feats, int cin, const float* pdf,
                     int64_t num_samples, const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                     const float* radii, const float* kernel_pts, int num_kernel_pts, float sigma, const float* weights,
                     int cout, float* out, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(kernel_pts && pdf && sigma > 0.f, "pccnn: kernel points or density missing, or sigma <= 0");
    KPDensityArgs args{kernel_pts, 1.0f / (sigma * sigma), pdf};
    return conv_forward<KPDensityArgs, GaussBasis>("pccnn", D, num_kernel_pts, args, num_pts, pts, feats, cin, num_samples,
                                                   samples, neighbors, start_ids, radii, 1, weights, cout, out, workspace,
                                                   workspace_bytes, (cudaStream_t)stream);
}

int pccnn_pccnn_conv_grads(int D, int64_t num_pts, const float* pts, const float* feats, int cin, const float* pdf,
                           int64_t num_samples, const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                           const float* radii, const float* kernel_pts, int num_kernel_pts, float sigma,
                           const float* weights, int cout, const float* in_grads, float* out_weight_grads,
                           float* out_feat_grads, float* out_kernel_pt_grads, float* out_pdf_grads, float* out_pt_grads,
                           float* out_sample_grads, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(kernel_pts && pdf && sigma > 0.f, "pccnn_grads: kernel points or density missing, or sigma <= 0");
    PCCNN_CHECK_ARG(out_kernel_pt_grads && out_pdf_grads && out_pt_grads && out_sample_grads, "pccnn_grads: null output");
    KPDensityArgs args{kernel_pts, 1.0f / (sigma * sigma), pdf};
    return conv_backward<KPDensityArgs, GaussBasis>(
        "pccnn_grads", D, num_kernel_pts, args, num_pts, pts, feats, cin, num_samples, samples, neighbors, start_ids, radii,
        1, weights, cout, in_grads, out_weight_grads, out_feat_grads, out_kernel_pt_grads, (size_t)num_kernel_pts * D,
        nullptr, 0, out_pdf_grads, out_pt_grads, out_sample_grads, workspace, workspace_bytes, (cudaStream_t)stream);
}

int pccnn_pccnn_conv_weight_var(int D, int64_t num_pts, const float* pts, const float* feats, int cin, const float* pdf,
                                int64_t num_samples, const float* samples, const int32_t* neighbors,
                                const int32_t* start_ids, const float* radii, const float* kernel_pts, int num_kernel_pts,
                                float sigma, float* out_variance, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(kernel_pts && pdf && sigma > 0.f, "pccnn_weight_variance: kernel points or density missing, or sigma <= 0");
    KPDensityArgs args{kernel_pts, 1.0f / (sigma * sigma), pdf};
    return conv_weight_var<KPDensityArgs, GaussBasis>("pccnn_weight_variance", D, num_kernel_pts, args, num_pts, pts, feats,
                                                      cin, num_samples, samples, neighbors, start_ids, radii, 0,
                                                      out_variance, workspace, workspace_bytes, (cudaStream_t)stream);
}

}  // extern "C"
