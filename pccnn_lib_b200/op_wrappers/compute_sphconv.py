import torch

from .. import ops


class ComputeSPHConv(torch.autograd.Function):
    """SPHConv operator with gradients (pccnn_lib/op_wrappers/compute_sphconv.py:7-52 of the reference): only the
    features and the weights receive gradients."""

    @staticmethod
    def forward(ctx, p_pts, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_radial_bins, p_azimuz_bins,
                p_polar_bins, p_conv_weights):
        ctx.save_for_backward(p_pts, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_radial_bins,
                              p_azimuz_bins, p_polar_bins, p_conv_weights)
        return ops.sph_conv(p_pts, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_radial_bins,
                            p_azimuz_bins, p_polar_bins, p_conv_weights)

    @staticmethod
    def backward(ctx, p_grads):
        pts, features, samples, neighbors, start_ids, radii, radial_bins, azimuz_bins, polar_bins, conv_weights = \
            ctx.saved_tensors
        weight_grads, feat_grads = ops.sph_conv_grads(pts, features, samples, neighbors, start_ids, radii, radial_bins,
                                                      azimuz_bins, polar_bins, conv_weights, p_grads.contiguous())
        return None, feat_grads, None, None, None, None, None, None, None, weight_grads


class ComputeSPHConvWeightVar(torch.autograd.Function):
    """pccnn_lib/op_wrappers/compute_sphconv.py:55-84 of the reference; not differentiable."""

    @staticmethod
    def forward(ctx, p_pts, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_radial_bins, p_azimuz_bins,
                p_polar_bins):
        return ops.sph_conv_weight_var(p_pts, p_features, p_samples, p_neighbors, p_start_ids, p_radii, p_radial_bins,
                                       p_azimuz_bins, p_polar_bins)

    @staticmethod
    def backward(ctx, p_grads):
        return None, None, None, None, None, None, None, None, None
