import math

import torch

from ...op_wrappers import ComputePointConv, ComputePointConvBasis, ComputePointConvWeightVar
from .IConvLayer import IConvLayer, IConvLayerFactory


class PointConv(IConvLayer):
    """PointConv (pccnn_lib/pc/layers/PointConv.py:10-214 of the reference): the basis of a pair is ReLU of an affine
    projection of its offset (optionally batch-normalised), weighted by a small MLP of the pair's inverse density
    relative to the densest neighbor of the sample; the convolution then runs on that [T, H] basis.
    The group-normalisation option of the reference needs its GroupNormalization layer, which is outside this
    package: p_use_gn raises."""

    def __init__(self, p_dims, p_in_features, p_out_features, p_hidden_size, p_constant_weight_var=True,
                 p_const_var_value=1.0, p_use_bn=False, p_use_gn=False, p_gn_size=32):
        super(PointConv, self).__init__(p_dims, p_in_features, p_out_features, p_constant_weight_var, p_const_var_value)
        if p_use_gn:
            raise NotImplementedError("PointConv with group normalisation needs the reference's GroupNormalization layer, "
                                      "which pccnn_lib_b200 does not carry")
        self.use_bn_ = p_use_bn
        self.use_gn_ = False
        self.gn_size_ = p_gn_size
        self.hidden_size_ = p_hidden_size
        self.init_proj_axis_ = False
        self.proj_axis_ = torch.nn.Parameter(torch.empty(self.num_dims_, self.hidden_size_))
        self.proj_bias_ = torch.nn.Parameter(torch.empty(1, self.hidden_size_))
        self.conv_weights_ = torch.nn.Parameter(torch.empty(self.hidden_size_ * self.feat_input_size_,
                                                            self.feat_output_size_))
        layers = [torch.nn.Linear(1, 16)]
        if self.use_bn_:
            layers.append(torch.nn.BatchNorm1d(16))
        layers += [torch.nn.ReLU(), torch.nn.Linear(16, 1)]
        if self.use_bn_:
            layers.append(torch.nn.BatchNorm1d(1))
        layers.append(torch.nn.Sigmoid())
        self.pdf_mlp_ = torch.nn.Sequential(*layers)
        if self.use_bn_:
            self.basis_bn_ = torch.nn.BatchNorm1d(p_hidden_size)
        self.reset_parameters()

    def reset_parameters(self):
        self.conv_weights_.data.normal_(0.0, math.sqrt(2.0 / (self.feat_input_size_ * self.hidden_size_)))
        self.proj_axis_.data.normal_(0.0, math.sqrt(1.0 / self.num_dims_))
        self.proj_bias_.data.fill_(0.0)

    def __compute_convolution__(self, p_pc_in, p_pc_out, p_in_features, p_radius, p_neighborhood):
        n0 = p_neighborhood.neighbors_[:, 0].to(torch.int64)
        n1 = p_neighborhood.neighbors_[:, 1].to(torch.int64)
        cur_pdf = torch.reciprocal(torch.index_select(p_pc_in.pts_unnorm_pdf_, 0, n0))
        # largest inverse density among the neighbors of every sample (torch_scatter.scatter_max in the reference)
        max_pdf = torch.zeros((p_pc_out.pts_.shape[0],), dtype=cur_pdf.dtype, device=cur_pdf.device)
        max_pdf = max_pdf.scatter_reduce(0, n1, cur_pdf, reduce="amax", include_self=False)
        cur_pdf = cur_pdf / torch.index_select(max_pdf, 0, n1)
        cur_pdf = self.pdf_mlp_(torch.reshape(cur_pdf, (-1, 1)))
        cur_radius = torch.ones_like(p_radius)
        warmup = self.wamup_state_ and self.use_const_variance_init_
        if warmup or self.init_proj_axis_:
            stdv = torch.sqrt(1.0 / (self.num_dims_ * p_radius[0] * p_radius[0]))
            self.proj_axis_.data.normal_(0.0, float(stdv))
            self.init_proj_axis_ = False
        basis_proj = ComputePointConvBasis.apply(p_pc_in.pts_, p_pc_out.pts_, p_neighborhood.neighbors_, cur_radius,
                                                 self.proj_axis_, self.proj_bias_)
        if self.use_bn_:
            basis_proj = self.basis_bn_(basis_proj)
        basis_proj = torch.nn.functional.relu(basis_proj) * cur_pdf
        if warmup:
            self.__warmup_weights__(ComputePointConvWeightVar.apply(basis_proj, p_in_features,
                                                                    p_neighborhood.neighbors_,
                                                                    p_neighborhood.start_ids_))
        return ComputePointConv.apply(basis_proj, p_in_features, p_neighborhood.neighbors_, p_neighborhood.start_ids_,
                                      self.conv_weights_)


class PointConvFactory(IConvLayerFactory):
    def __init__(self, p_num_basis, p_const_var_w_init=False, p_const_var_value=1.0, p_use_bn=False, p_use_gn=False,
                 p_gn_size=32):
        self.use_gn_ = p_use_gn
        self.use_bn_ = p_use_bn and not p_use_gn
        self.gn_size_ = p_gn_size
        super(PointConvFactory, self).__init__(p_num_basis, p_const_var_w_init, p_const_var_value)

    def create_conv_layer(self, p_dims, p_in_features, p_out_features):
        layer = PointConv(p_dims, p_in_features, p_out_features, self.num_basis_, self.conv_var_w_init_,
                          self.const_var_value_, self.use_bn_, self.use_gn_, self.gn_size_)
        self.conv_list_.append(layer)
        return layer
