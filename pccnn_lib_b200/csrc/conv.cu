// KPConv / MCConv forward: neighbor gather x basis projection, then the tensor-core contraction.
//
// Restates pccnn_lib_ops/pcconvs/kpconv.cu:32-60 and mcconv.cu:32-71 of phermosilla/pccnn_lib with
// their stages pt_diff (shared/pt_diff.cu:27-49), kernel_pts_basis (shared/kernel_pts_basis.cu:23-39),
// mlp_basis (shared/mlp_basis.cu:27-48) and feat_basis_proj (shared/feat_basis_proj.cu:30-129):
//     d_t      = (pts[n0(t)] - samples[n1(t)]) * (1 / radii)
//     b[t, k]  = clamp(1 - |kp_k - d_t| / sigma, 0, 1)                  (KPConv)
//              = leaky_relu_{0.2}(d_t . A[:, k] + bias[k]) / pdf[n0(t)]  (MCConv)
//     P[m,c,k] = sum_{t in seg(m)} F[n0(t), c] * b[t, k]
//     out      = P.reshape(M, Cin*K) @ W
//
// Design.  The reference runs ~10 elementwise launches that materialise [T, D], [T, K, D] and
// [T, K] tensors, then a 64-thread block per (sample, 8 channels) that re-reads the basis row
// Cin/8 times.  Here one kernel does everything up to P: a warp owns a sample, its lanes first
// act as 32 neighbors (offset + all K basis values per lane, parked in shared memory), then as
// 32 channels x CPL, streaming the neighbors' feature rows with coalesced 128-byte loads and
// broadcasting the basis row from shared memory; CPL * K = 64 fp32 accumulators per lane, so the
// basis is evaluated once per pair for up to 32 * CPL channels.  P leaves the kernel as bf16
// hi + lo parts in the layout the contraction's TMA loads expect, and out = P @ W runs on
// tcgen05 (gemm.cu), in sample chunks so the scratch stays bounded.
#include "conv_impl.cuh"

namespace pccnn {
thread_local cudaEvent_t g_weight_grads_event = nullptr;
int g_conv_path = 0;
}


using namespace pccnn;

extern "C" {

size_t pccnn_conv_workspace_bytes(int64_t num_pts, int64_t num_samples, int cin, int basis_size, int cout) {
    return conv_layout(num_pts < 0 ? 0 : num_pts, num_samples < 0 ? 0 : num_samples, cin, basis_size, cout).total;
}

int pccnn_kp_conv(int D, int64_t num_pts, const float* pts, const float* feats, int cin, int64_t num_samples,
                  const float* samples, const int32_t* neighbors, const int32_t* start_ids, const float* radii,
                  const float* kernel_pts, int num_kernel_pts, float sigma, const float* weights, int cout,
                  float* out, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(kernel_pts && sigma > 0.f, "kp_conv: kernel points missing or sigma <= 0");
    KPBasisArgs args{kernel_pts, 1.0f / sigma};
    return conv_forward<KPBasisArgs, KPBasis>("kp_conv", D, num_kernel_pts, args, num_pts, pts, feats, cin, num_samples,
                                              samples, neighbors, start_ids, radii, 1, weights, cout, out, workspace,
                                              workspace_bytes, (cudaStream_t)stream);
}

size_t pccnn_kp_conv_grid_workspace_bytes(int64_t num_pts, int64_t num_samples, int cin, int num_kernel_pts, int cout) {
    return conv_grid_layout(num_pts < 0 ? 0 : num_pts, num_samples < 0 ? 0 : num_samples, cin, num_kernel_pts, cout).total;
}

int pccnn_kp_conv_grid(int64_t num_pts, const float* sorted_pts, const int64_t* sorted_keys, const int64_t* pt_index_map,
                       const void* feats, int feats_are_bf16, int cin, int64_t num_samples, const float* samples,
                       const int64_t* sample_keys, const int32_t* grid_ds, const int32_t* grid_size, const float* radii,
                       const float* kernel_pts, int num_kernel_pts, float sigma, const void* weights, int cout, void* out,
                       void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(kernel_pts && sigma > 0.f, "kp_conv_grid: kernel points missing or sigma <= 0");
    KPBasisArgs args{kernel_pts, 1.0f / sigma};
    return conv_forward_grid<KPBasisArgs, KPBasis>("kp_conv_grid", num_kernel_pts, args, num_pts, sorted_pts, sorted_keys,
                                                   pt_index_map, feats, feats_are_bf16, cin, num_samples, samples, sample_keys,
                                                   grid_ds, grid_size, radii, weights, cout, out, workspace, workspace_bytes,
                                                   (cudaStream_t)stream);
}

int pccnn_kp_conv_bf16(int D, int64_t num_pts, const float* pts, const void* feats_bf16, int cin, int64_t num_samples,
                       const float* samples, const int32_t* neighbors, const int32_t* start_ids, const float* radii,
                       const float* kernel_pts, int num_kernel_pts, float sigma, const void* weights_bf16, int cout,
                       void* out_bf16, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(kernel_pts && sigma > 0.f, "kp_conv_bf16: kernel points missing or sigma <= 0");
    KPBasisArgs args{kernel_pts, 1.0f / sigma};
    return conv_forward<KPBasisArgs, KPBasis, true>("kp_conv_bf16", D, num_kernel_pts, args, num_pts, pts, feats_bf16, cin,
                                              num_samples, samples, neighbors, start_ids, radii, 1, weights_bf16, cout,
                                              out_bf16, workspace, workspace_bytes, (cudaStream_t)stream, true);
}

int pccnn_mc_conv(int D, int64_t num_pts, const float* pts, const float* pdf, const float* feats, int cin,
                  int64_t num_samples, const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                  const float* radii, const float* axis, const float* bias, int hidden, int num_mlps,
                  const float* weights, int cout, float* out, void* workspace, size_t workspace_bytes,
                  void* stream) {
    PCCNN_CHECK_ARG(pdf && axis && bias, "mc_conv: null pointer");
    MLPBasisArgs args{axis, bias, pdf};
    return conv_forward<MLPBasisArgs, MLPBasis>("mc_conv", D, hidden, args, num_pts, pts, feats, cin, num_samples,
                                                samples, neighbors, start_ids, radii, num_mlps, weights, cout, out,
                                                workspace, workspace_bytes, (cudaStream_t)stream);
}

#ifdef PCCNN_TC_PROFILE
int pccnn_debug_tc_profile(long long* out16) {
    PCCNN_CUDA(cudaDeviceSynchronize());
    PCCNN_CUDA(cudaMemcpyFromSymbol(out16, g_tc_prof, sizeof(long long) * 16));
    return PCCNN_OK;
}
#endif

int pccnn_conv_set_path(int path) {
    PCCNN_CHECK_ARG(path == 0 || path == 1, "conv_set_path: 0 (tensor-core pair kernels where they apply) or 1 (CUDA cores)");
    g_conv_path = path;
    return PCCNN_OK;
}

int pccnn_conv_grads_set_weight_grads_event(void* event) {
    g_weight_grads_event = (cudaEvent_t)event;
    return PCCNN_OK;
}

size_t pccnn_conv_weight_var_workspace_bytes(int64_t num_pts, int64_t num_samples, int cin, int basis_size) {
    return conv_weight_var_workspace(num_pts < 0 ? 0 : num_pts, num_samples < 0 ? 0 : num_samples, cin, basis_size);
}

int pccnn_kp_conv_weight_var(int D, int64_t num_pts, const float* pts, const float* feats, int cin, int64_t num_samples,
                             const float* samples, const int32_t* neighbors, const int32_t* start_ids, const float* radii,
                             const float* kernel_pts, int num_kernel_pts, float sigma, float* out_variance,
                             void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(kernel_pts && sigma > 0.f, "kp_conv_weight_var: kernel points missing or sigma <= 0");
    KPBasisArgs args{kernel_pts, 1.0f / sigma};
    return conv_weight_var<KPBasisArgs, KPBasis>("kp_conv_weight_var", D, num_kernel_pts, args, num_pts, pts, feats, cin,
                                                 num_samples, samples, neighbors, start_ids, radii, 0, out_variance,
                                                 workspace, workspace_bytes, (cudaStream_t)stream);
}

int pccnn_mc_conv_weight_var(int D, int64_t num_pts, const float* pts, const float* pdf, const float* feats, int cin,
                             int64_t num_samples, const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                             const float* radii, const float* axis, const float* bias, int hidden, float* out_variance,
                             void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(pdf && axis && bias, "mc_conv_weight_var: null pointer");
    MLPBasisArgs args{axis, bias, pdf};
    return conv_weight_var<MLPBasisArgs, MLPBasis>("mc_conv_weight_var", D, hidden, args, num_pts, pts, feats, cin,
                                                   num_samples, samples, neighbors, start_ids, radii, 0, out_variance,
                                                   workspace, workspace_bytes, (cudaStream_t)stream);
}

size_t pccnn_conv_grads_workspace_bytes(int64_t num_pts, int64_t num_samples, int cin, int basis_size, int cout) {
    return conv_backward_layout(num_pts < 0 ? 0 : num_pts, num_samples < 0 ? 0 : num_samples, cin, basis_size, cout).total;
}

int pccnn_kp_conv_grads(int D, int64_t num_pts, const float* pts, const float* feats, int cin, int64_t num_samples,
                        const float* samples, const int32_t* neighbors, const int32_t* start_ids, const float* radii,
                        const float* kernel_pts, int num_kernel_pts, float sigma, const float* weights, int cout,
                        const float* in_grads, float* out_weight_grads, float* out_feat_grads,
                        float* out_kernel_pt_grads, float* out_pt_grads, float* out_sample_grads, void* workspace,
                        size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(kernel_pts && sigma > 0.f, "kp_conv_grads: kernel points missing or sigma <= 0");
    KPBasisArgs args{kernel_pts, 1.0f / sigma};
    return conv_backward<KPBasisArgs, KPBasis>(
        "kp_conv_grads", D, num_kernel_pts, args, num_pts, pts, feats, cin, num_samples, samples, neighbors, start_ids,
        radii, 1, weights, cout, in_grads, out_weight_grads, out_feat_grads, out_kernel_pt_grads,
        (size_t)num_kernel_pts * D, nullptr, 0, nullptr, out_pt_grads, out_sample_grads, workspace, workspace_bytes,
        (cudaStream_t)stream);
}

int pccnn_mc_conv_grads(int D, int64_t num_pts, const float* pts, const float* pdf, const float* feats, int cin,
                        int64_t num_samples, const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                        const float* radii, const float* axis, const float* bias, int hidden, int num_mlps,
                        const float* weights, int cout, const float* in_grads, float* out_weight_grads,
                        float* out_feat_grads, float* out_axis_grads, float* out_bias_grads, float* out_pdf_grads,
                        float* out_pt_grads, float* out_sample_grads, void* workspace, size_t workspace_bytes,
                        void* stream) {
    PCCNN_CHECK_ARG(pdf && axis && bias && out_bias_grads && out_pdf_grads, "mc_conv_grads: null pointer");
    MLPBasisArgs args{axis, bias, pdf};
    return conv_backward<MLPBasisArgs, MLPBasis>(
        "mc_conv_grads", D, hidden, args, num_pts, pts, feats, cin, num_samples, samples, neighbors, start_ids, radii,
        num_mlps, weights, cout, in_grads, out_weight_grads, out_feat_grads, out_axis_grads, (size_t)D * hidden,
        out_bias_grads, (size_t)hidden, out_pdf_grads, out_pt_grads, out_sample_grads, workspace, workspace_bytes,
        (cudaStream_t)stream);
}

}  // extern "C"
