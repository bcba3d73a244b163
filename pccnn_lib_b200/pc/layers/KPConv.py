import math

import numpy as np
import torch

from ... import ops
from ...op_wrappers import ComputeKPConv, ComputeKPConvWeightVar
from ...py_utils.pc_utils import rotate_pc_3d
from .IConvLayer import IConvLayer, IConvLayerFactory
from .kernel_points.kernel_points import kernel_pts_dict


def prepare_kernel_points(p_dims, p_num_kernel_pts, p_table=None, p_sigma_scale=1.0, p_rotation_seed=15):
    """Kernel points and sigma exactly as pccnn_lib/pc/layers/KPConv.py:45-57 of the reference
    prepares them: normalise by the largest norm, rotate 3-D sets with RandomState(15), divide by
    (1 + smallest shell norm); sigma = smallest shell norm / (1 + smallest shell norm).
    KPConvN and PCCNN of the reference differ only in the factor on sigma (2.0 and 0.4) and in seeding the
    rotation with the clock (KPConvN.py:46-57, PCCNN.py:46-57).  Returns (float32 array [K, dims], float)."""
    table = kernel_pts_dict[str(p_dims) + "_" + str(p_num_kernel_pts)] if p_table is None else p_table
    pts = np.asarray(table).astype(np.float32)
    dist = np.linalg.norm(pts, axis=-1).astype(np.float32)
    max_dist = np.amax(dist)
    dist = dist / max_dist
    pts = pts / max_dist
    min_distance = np.amin(dist[1:])
    if pts.shape[-1] == 3:
        pts, _ = rotate_pc_3d(np.random.RandomState(p_rotation_seed), pts)
    pts = pts.astype(np.float32)
    return pts / (1.0 + min_distance), float((min_distance * p_sigma_scale) / (1.0 + min_distance))


class KPConv(IConvLayer):
    """Kernel point convolution (pccnn_lib/pc/layers/KPConv.py:11-146 of the reference).
    Buffers ``kernel_pts_`` / ``sigma_`` and parameter ``conv_weights_`` [K * Cin, Cout] keep the
    reference's names, so state dicts interchange."""

    def __init__(self, p_dims, p_in_features, p_out_features, p_num_kernel_pts, p_constant_weight_var=True,
                 p_const_var_value=1.0):
        super(KPConv, self).__init__(p_dims, p_in_features, p_out_features, p_constant_weight_var, p_const_var_value)
        self.num_kernel_pts_ = p_num_kernel_pts
        kernel_pts, sigma = prepare_kernel_points(p_dims, p_num_kernel_pts)
        self.register_buffer('kernel_pts_', torch.from_numpy(kernel_pts))
        self.register_buffer('sigma_', torch.tensor(sigma))
        self.sigma_cpu_ = None
        self.conv_weights_ = torch.nn.Parameter(
            torch.empty(self.num_kernel_pts_ * self.feat_input_size_, self.feat_output_size_))
        self.reset_parameters()

    def reset_parameters(self):
        stdv = math.sqrt(2.0 / (self.feat_input_size_ * self.num_kernel_pts_))
        self.conv_weights_.data.normal_(0.0, stdv)

    def __compute_convolution__(self, p_pc_in, p_pc_out, p_in_features, p_radius, p_neighborhood):
        if self.sigma_cpu_ is None:
            self.sigma_cpu_ = self.sigma_.item()
        if getattr(p_neighborhood, "neighbors_", 0) is None:
            # a GridNeighborhood: no list exists, the convolution searches the grid in its own kernel (inference only)
            if torch.is_grad_enabled() and (p_in_features.requires_grad or self.conv_weights_.requires_grad):
                raise RuntimeError("a GridNeighborhood carries no neighbor list, which the gradient operators need: "
                                   "use a Neighborhood for training, or run the layer under torch.no_grad()")
            grid = p_neighborhood.grid_
            return ops.kp_conv_grid(grid.sorted_pts_, grid.sorted_cell_ids_, grid.sorted_ids_, p_in_features,
                                    p_pc_out.pts_, p_neighborhood.sample_cell_ids_, grid.grid_ds_, grid.num_cells_,
                                    grid.cell_size_, self.kernel_pts_, self.sigma_cpu_, self.conv_weights_.to(p_in_features.dtype))
        if self.wamup_state_ and self.use_const_variance_init_:
            self.__warmup_weights__(ComputeKPConvWeightVar.apply(
                p_pc_in.pts_, p_in_features, p_pc_out.pts_, p_neighborhood.neighbors_, p_neighborhood.start_ids_, p_radius,
                self.kernel_pts_, self.sigma_cpu_))
        return ComputeKPConv.apply(p_pc_in.pts_, p_in_features, p_pc_out.pts_, p_neighborhood.neighbors_,
                                   p_neighborhood.start_ids_, p_radius, self.kernel_pts_, self.sigma_cpu_,
                                   self.conv_weights_)


class KPConvFactory(IConvLayerFactory):
    def __init__(self, p_num_kernel_pts, p_const_var_w_init=False, p_const_var_value=1.0):
        super(KPConvFactory, self).__init__(p_num_kernel_pts, p_const_var_w_init, p_const_var_value)

    def create_conv_layer(self, p_dims, p_in_features, p_out_features):
        layer = KPConv(p_dims, p_in_features, p_out_features, self.num_basis_, self.conv_var_w_init_,
                       self.const_var_value_)
        self.conv_list_.append(layer)
        return layer
