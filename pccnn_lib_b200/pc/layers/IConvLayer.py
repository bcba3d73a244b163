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
        """Variance-aware warm-up initialisation needs the *_weight_var operators, which are not
        part of this package; the flag is kept for interface compatibility."""
        if p_init_warmup_state and self.use_const_variance_init_:
            raise NotImplementedError("variance-aware warm-up initialisation is not available in pccnn_lib_b200")
        self.wamup_state_ = p_init_warmup_state

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
    """Factory interface (pccnn_lib/pc/layers/IConvLayer.py:160-186 of the reference)."""

    def __init__(self, p_constant_weight_var=False, p_const_var_value=1.0):
        self.use_const_variance_init_ = p_constant_weight_var
        self.conv_var_value_ = p_const_var_value
        self.conv_list_ = []

    def update_conv_const_var_value(self, p_const_var_value):
        self.conv_var_value_ = p_const_var_value

    @abstractmethod
    def create_conv_layer(self, p_dims, p_in_features, p_out_features):
        pass
