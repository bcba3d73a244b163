import torch

from .. import ops


class ComputePointConvBasis(torch.autograd.Function):
    """Affine projection of the normalised neighbor offsets, [T, H]
    (pccnn_lib/op_wrappers/compute_pointconv.py:6-54 of the reference).  backward:
    (pts, samples, None, None, axis_proj, axis_bias)."""

    @staticmethod
    def forward(ctx, p_pts, p_samples, p_neighbors, p_radii, p_axis_proj, p_axis_bias):
        ctx.save_for_backward(p_pts, p_samples, p_neighbors, p_radii, p_axis_proj, p_axis_bias)
        return ops.point_conv_basis(p_pts, p_radii, p_samples, p_neighbors, p_axis_proj, p_axis_bias)

    @staticmethod
    def backward(ctx, p_grads):
        pts, samples, neighbors, radii, axis_proj, axis_bias = ctx.saved_tensors
        pt_grads, sample_grads, axis_grad, bias_grad = ops.point_conv_basis_grads(
            pts, radii, samples, neighbors, axis_proj, axis_bias, p_grads.contiguous())
        return pt_grads, sample_grads, None, None, axis_grad, bias_grad.reshape(axis_bias.shape)


class ComputePointConv(torch.autograd.Function):
    """Convolution on a caller-made basis (pccnn_lib/op_wrappers/compute_pointconv.py:57-102 of the reference).
    backward: (basis, features, None, None, weights)."""

    @staticmethod
    def forward(ctx, p_basis_proj, p_features, p_neighbors, p_start_ids, p_conv_weights):
        ctx.save_for_backward(p_basis_proj, p_features, p_neighbors, p_start_ids, p_conv_weights)
        return ops.point_conv(p_basis_proj, p_features, p_neighbors, p_start_ids, p_conv_weights)

    @staticmethod
    def backward(ctx, p_grads):
        basis_proj, features, neighbors, start_ids, conv_weights = ctx.saved_tensors
        weights_grads, feat_grads, basis_grads = ops.point_conv_grads(basis_proj, features, neighbors, start_ids,
                                                                      conv_weights, p_grads.contiguous())
        return basis_grads, feat_grads, None, None, weights_grads


class ComputePointConvWeightVar(torch.autograd.Function):
    """pccnn_lib/op_wrappers/compute_pointconv.py:105-130 of the reference; not differentiable."""

    @staticmethod
    def forward(ctx, p_basis, p_features, p_neighbors, p_start_ids):
        return ops.point_conv_weight_var(p_basis, p_features, p_neighbors, p_start_ids)

    @staticmethod
    def backward(ctx, p_grads):
        return None, None, None, None
