import torch

from .. import ops


class Neighborhood(object):
    """Radius neighborhood of every sample in the points of a grid
    (pccnn_lib/pc/Neighborhood.py:10-53 of the reference).

    ``neighbors_`` [T, 2] int32 rows (ORIGINAL point index, sample index), grouped by sample,
    ascending sorted position inside a sample; ``start_ids_`` [M] int32 inclusive end offsets.
    The search radius is the grid's cell size.  The mapping from sorted positions back to
    original indices happens inside the search kernel.
    """

    def __init__(self, p_grid, p_samples, p_max_neighbors=0):
        self.grid_ = p_grid
        self.samples_ = p_samples
        with torch.no_grad():
            grid = self.grid_
            if grid.grid_ds_ is None:
                grid.compute_cell_ids()
                grid.build_ds()
            # keys carry no gradient: the operator is called directly, without the autograd wrapper
            sample_cell_ids = ops.compute_keys(self.samples_.pts_.detach(), self.samples_.batch_ids_,
                                               grid.bounding_box_.min_, grid.num_cells_, grid.cell_size_)
            self.neighbors_, self.start_ids_ = ops.find_neighbors(
                grid.sorted_pts_, grid.sorted_cell_ids_, self.samples_.pts_.detach(), sample_cell_ids,
                grid.grid_ds_, grid.num_cells_, grid.cell_size_, p_max_neighbors, pt_index_map=grid.sorted_ids_,
                key_bits=grid.key_bits())
            # The uncapped neighborhood of a point cloud in itself holds every pair in both rows; operators that can use
            # that (the gradient of the density) read the mark from the list.
            self.full_self_ = self.samples_ is grid.pointcloud_ and not p_max_neighbors
            self.neighbors_._pccnn_full_self = self.full_self_

    def __repr__(self):
        return "### Neighbors:\n{}\n### Start indices:\n{}".format(self.neighbors_, self.start_ids_)


class GridNeighborhood(object):
    """The neighborhood of every sample in the points of a grid, WITHOUT the list: it holds the grid and the samples'
    cell keys, and the convolution that receives it searches the grid inside its own kernel (ops.kp_conv_grid).
    No counterpart in the reference, whose Neighborhood always materialises ``neighbors_`` [T, 2].  Inference only
    (the gradient operators read a list): KPConv accepts it when no gradient is required; 3-D points, search radius
    = the grid's cell size."""

    def __init__(self, p_grid, p_samples):
        self.grid_ = p_grid
        self.samples_ = p_samples
        self.neighbors_ = None
        self.start_ids_ = None
        with torch.no_grad():
            grid = self.grid_
            if grid.grid_ds_ is None:
                grid.compute_cell_ids()
                grid.build_ds()
            self.sample_cell_ids_ = ops.compute_keys(self.samples_.pts_.detach(), self.samples_.batch_ids_,
                                                     grid.bounding_box_.min_, grid.num_cells_, grid.cell_size_)
