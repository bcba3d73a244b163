import torch

from .. import ops


class ComputeKPConv(torch.autograd.Function):
    """KPConv operator with gradients (pccnn_lib/op_wrappers/compute_kpconv.py:10-73 of the reference).
    backward returns gradients in the positional order of forward's inputs:
    (pts, features, samples, None, None, None, kernel_pts, None, weights)."""

    @staticmethod
    def forward(ctx, p_pts, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts, p_sigma,
                p_conv_weights):
        ctx.save_for_backward(p_pts, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts,
                              p_conv_weights)
        ctx.sigma_ = p_sigma
        return ops.kp_conv(p_pts, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts, p_sigma,
                           p_conv_weights)

    @staticmethod
    def backward(ctx, p_grads):
        pts, features, samples, neighbors, start_ids, radii, kernel_pts, conv_weights = ctx.saved_tensors
        weight_grads, feat_grads, kernel_pts_grads, pt_grads, sample_grads = ops.kp_conv_grads(
            pts, features, samples, neighbors, start_ids, radii, kernel_pts, ctx.sigma_, conv_weights,
            p_grads.contiguous())
        return pt_grads, feat_grads, sample_grads, None, None, None, kernel_pts_grads, None, weight_grads


class ComputeKPConvWeightVar(torch.autograd.Function):
    """Weight variance a KPConv layer should be initialised with on this batch
    (pccnn_lib/op_wrappers/compute_kpconv.py:76-116 of the reference); not differentiable."""

    @staticmethod
    def forward(ctx, p_pts, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts, p_sigma):
        return ops.kp_conv_weight_var(p_pts, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts,
                                      p_sigma)

    @staticmethod
    def backward(ctx, p_grads):
        return None, None, None, None, None, None, None, None
