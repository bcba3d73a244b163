import torch

from .. import ops


class ComputePCCNN(torch.autograd.Function):
    """PCCNN operator with gradients (pccnn_lib/op_wrappers/compute_pccnn.py:7-66 of the reference).  The wrapper
    takes the density before the features, the operator the other way round, as in the reference.  backward:
    (pts, pt_pdf, features, samples, None, None, None, kernel_pts, None, weights)."""

    @staticmethod
    def forward(ctx, p_pts, p_pt_pdf, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts, p_sigma,
                p_conv_weights):
        ctx.save_for_backward(p_pts, p_pt_pdf, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts,
                              p_conv_weights)
        ctx.sigma_ = p_sigma
        return ops.pccnn(p_pts, p_features, p_pt_pdf, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts,
                         p_sigma, p_conv_weights)

    @staticmethod
    def backward(ctx, p_grads):
        pts, pt_pdf, features, samples, neighbors, start_ids, radii, kernel_pts, conv_weights = ctx.saved_tensors
        weight_grads, feat_grads, kernel_pts_grads, pt_pdf_grads, pt_grads, sample_grads = ops.pccnn_grads(
            pts, features, pt_pdf, samples, neighbors, start_ids, radii, kernel_pts, ctx.sigma_, conv_weights,
            p_grads.contiguous())
        return pt_grads, pt_pdf_grads, feat_grads, sample_grads, None, None, None, kernel_pts_grads, None, weight_grads


class ComputePCCNNWeightVar(torch.autograd.Function):
    """pccnn_lib/op_wrappers/compute_pccnn.py:69-112 of the reference; not differentiable."""

    @staticmethod
    def forward(ctx, p_pts, p_pt_pdf, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_kernel_pts, p_sigma):
        return ops.pccnn_weight_variance(p_pts, p_features, p_pt_pdf, p_samples, p_neighbors, p_start_ids, p_radii,
                                         p_kernel_pts, p_sigma)

    @staticmethod
    def backward(ctx, p_grads):
        return None, None, None, None, None, None, None, None, None
