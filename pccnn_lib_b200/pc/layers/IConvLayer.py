import math
from abc import ABC, abstractmethod

import torch


class IConvLayer(torch.nn.Module, ABC):
    """Base class of the point convolutions (pccnn_lib/pc/layers/IConvLayer.py:7-157 of the reference).

    forward(pc_in, pc_out, features, radius, neighborhood=None, max_neighs=0) returns the output
    features, and also the neighborhood it built when none was passed in.
    """

    def __init__(self, p_dims, p_in_features, p_out_features, p_constant_weight_var=True, p_const_var_value=1.0):
        super(IConvLayer, self).__init__()
        self.num_dims_ = p_dims
        self.feat_input_size_ = p_in_features
        self.feat_output_size_ = p_out_features
        self.wamup_state_ = False
        self.use_const_variance_init_ = p_constant_weight_var
        self.out_constant_variance_ = p_const_var_value
        self.accum_weight_var_ = 0.0
        self.accum_weight_var_counter_ = 1.0

    def set_init_warmup_state(self, p_init_warmup_state):
        """While the flag is set (and the layer was built with the constant-variance initialisation), every forward
        pass accumulates the weight variance its batch asks for (the *_weight_var operators) and re-draws the
        weights with it (pccnn_lib/pc/layers/IConvLayer.py:47-57, KPConv.py:103-116 of the reference)."""
        self.wamup_state_ = p_init_warmup_state

    def __warmup_weights__(self, p_variance):
        """Shared tail of the layers' warm-up branch: accumulate 1 / variance, re-draw the weights."""
        self.__update_weight_var__(1.0 / p_variance.item())
        stdv = math.sqrt(self.out_constant_variance_ / self.accum_weight_var_)
        self.conv_weights_.data.normal_(0.0, stdv)

    def __update_weight_var__(self, p_new_var):
        self.accum_weight_var_ += (p_new_var - self.accum_weight_var_) / self.accum_weight_var_counter_
        self.accum_weight_var_counter_ += 1.0

    @abstractmethod
    def __compute_convolution__(self, p_pc_in, p_pc_out, p_in_features, p_radius, p_neighborhood):
        pass

    def __create_neighborhood__(self, p_pc_in, p_pc_out, p_radius, p_max_neighs):
        from ..BoundingBox import BoundingBox
        from ..Grid import Grid
        from ..Neighborhood import Neighborhood
        bb = BoundingBox(p_pc_in)
        grid = Grid(p_pc_in, bb, p_radius)
        grid.compute_cell_ids()
        grid.build_ds()
        return Neighborhood(grid, p_pc_out, p_max_neighs)

    def forward(self, p_pc_in, p_pc_out, p_in_features, p_radius, p_neighborhood=None, p_max_neighs=0):
        if not torch.is_tensor(p_radius):
            radius = torch.as_tensor(p_radius, device=p_pc_in.pts_.device).to(torch.float32)
        else:
            radius = p_radius
        neighborhood = p_neighborhood
        if neighborhood is None:
            neighborhood = self.__create_neighborhood__(p_pc_in, p_pc_out, radius, p_max_neighs)
        out_features = self.__compute_convolution__(p_pc_in, p_pc_out, p_in_features, radius, neighborhood)
        if p_neighborhood is None:
            return out_features, neighborhood
        return out_features


class IConvLayerFactory(ABC):
    """Factory interface (pccnn_lib/pc/layers/IConvLayer.py:160-215 of the reference): number of basis functions,
    whether the layers use the constant-variance initialisation, and the list of the layers created."""

    def __init__(self, p_num_basis, p_const_var_w_init, p_const_var_value=1.0):
        super(IConvLayerFactory, self).__init__()
        self.num_basis_ = p_num_basis
        self.conv_var_w_init_ = p_const_var_w_init
        self.const_var_value_ = p_const_var_value
        self.conv_list_ = []

    def set_init_warmup_state_convs(self, p_state):
        for cur_conv in self.conv_list_:
            cur_conv.set_init_warmup_state(p_state)

    def define_num_basis(self, p_num_basis):
        self.num_basis_ = p_num_basis

    def update_conv_const_var_value(self, p_const_var_value):
        self.const_var_value_ = p_const_var_value

    @abstractmethod
    def create_conv_layer(self, p_dims, p_in_features, p_out_features):
        pass
