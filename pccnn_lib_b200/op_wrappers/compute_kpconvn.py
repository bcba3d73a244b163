import torch

from .. import ops


class ComputeKPConvN(torch.autograd.Function):
    """KPConvN operator with gradients (pccnn_lib/op_wrappers/compute_kpconvn.py:7-75 of the reference).
    backward returns gradients in the positional order of forward's inputs:
    (pts, None, features, samples, None, None, None, kernel_pts, None, weights) -- the reference gives the density
    no gradient."""

    @staticmethod
    def forward(ctx, p_pts, p_pdfs, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts, p_sigma,
                p_conv_weights):
        ctx.save_for_backward(p_pts, p_pdfs, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts,
                              p_conv_weights)
        ctx.sigma_ = p_sigma
        return ops.kp_conv_n(p_pts, p_pdfs, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts,
                             p_sigma, p_conv_weights)

    @staticmethod
    def backward(ctx, p_grads):
        pts, pdfs, features, samples, neighbors, start_ids, radii, kernel_pts, conv_weights = ctx.saved_tensors
        weight_grads, feat_grads, kernel_pts_grads, pt_grads, sample_grads = ops.kp_conv_n_grads(
            pts, pdfs, features, samples, neighbors, start_ids, radii, kernel_pts, ctx.sigma_, conv_weights,
            p_grads.contiguous())
        return pt_grads, None, feat_grads, sample_grads, None, None, None, kernel_pts_grads, None, weight_grads


class ComputeKPConvNWeightVar(torch.autograd.Function):
    """pccnn_lib/op_wrappers/compute_kpconvn.py:78-120 of the reference; not differentiable."""

    @staticmethod
    def forward(ctx, p_pts, p_pdfs, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts, p_sigma):
        return ops.kp_conv_n_weight_var(p_pts, p_pdfs, p_features, p_samples, p_neighbors, p_start_ids, p_radii,
                                        p_kernel_pts, p_sigma)

    @staticmethod
    def backward(ctx, p_grads):
        return None, None, None, None, None, None, None, None, None
