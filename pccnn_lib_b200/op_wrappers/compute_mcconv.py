import torch

from .. import ops


class ComputeMCConv(torch.autograd.Function):
    """MCConv operator with gradients (pccnn_lib/op_wrappers/compute_mcconv.py:10-75 of the reference).
    backward returns (pts, pdf, features, samples, None, None, None, axis, bias, weights)."""

    @staticmethod
    def forward(ctx, p_pts, p_pt_pdf, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_axis_proj,
                p_axis_bias, p_conv_weights):
        ctx.save_for_backward(p_pts, p_pt_pdf, p_features, p_samples, p_neighbors, p_start_ids, p_radii,
                              p_axis_proj, p_axis_bias, p_conv_weights)
        return ops.mc_conv(p_pts, p_pt_pdf, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_axis_proj,
                           p_axis_bias, p_conv_weights)

    @staticmethod
    def backward(ctx, p_grads):
        (pts, pt_pdf, features, samples, neighbors, start_ids, radii, axis_proj, axis_bias,
         conv_weights) = ctx.saved_tensors
        (weight_grads, feat_grads, axis_grad, bias_grad, pdf_grad, pt_grads, sample_grads) = ops.mc_conv_grads(
            pts, pt_pdf, features, samples, neighbors, start_ids, radii, axis_proj, axis_bias, conv_weights,
            p_grads.contiguous())
        return pt_grads, pdf_grad, feat_grads, sample_grads, None, None, None, axis_grad, bias_grad, weight_grads


class ComputeMCConvWeightVar(torch.autograd.Function):
    """Weight variance an MCConv layer should be initialised with on this batch
    (pccnn_lib/op_wrappers/compute_mcconv.py:78-119 of the reference); not differentiable."""

    @staticmethod
    def forward(ctx, p_pts, p_pt_pdf, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_axis_proj,
                p_axis_bias):
        return ops.mc_conv_weight_var(p_pts, p_pt_pdf, p_features, p_samples, p_neighbors, p_start_ids, p_radii,
                                      p_axis_proj, p_axis_bias)

    @staticmethod
    def backward(ctx, p_grads):
        return None, None, None, None, None, None, None, None, None
