import torch

from .BoundingBox import BoundingBox
from .Grid import Grid
from .. import ops


class PointPooling(object):
    """Pooling of a point cloud (pccnn_lib/pc/PointPooling.py:18-102 of the reference).

    ``poisson_disk``: greedy Poisson-disk subset with the given radii; ``pooling_ids_`` are the
    original indices of the kept points (int64), in ascending sorted position.
    ``cell_average``: one output per occupied grid cell; ``pooling_ids_`` maps points to cells.
    """

    def __init__(self, p_point_cloud, p_radii, p_method="poisson_disk"):
        self.point_cloud_ = p_point_cloud
        self.radii_ = p_radii
        self.method_ = p_method
        with torch.no_grad():
            bb = BoundingBox(self.point_cloud_)
            grid = Grid(self.point_cloud_, bb, self.radii_)
            grid.compute_cell_ids()
            grid.build_ds()
            if p_method == "poisson_disk":
                # the reference searches the full self-neighborhood and hands it to the sampling operator;
                # the grid-based operator makes the same selection without that list
                sampled = ops.poisson_disk_sampling_grid(grid.sorted_pts_, grid.sorted_cell_ids_, grid.grid_ds_,
                                                         grid.num_cells_, grid.cell_size_)
                self.pooling_ids_ = torch.index_select(grid.sorted_ids_, 0, sampled.reshape(-1))
            elif p_method == "cell_average":
                unique_ids, inverse_ids = torch.unique(grid.cell_ids_, return_inverse=True)
                self.pooling_ids_ = inverse_ids
                self.num_pooling_pts_ = unique_ids.shape[0]
            else:
                raise RuntimeError("unknown pooling method %r" % (p_method,))

    def pool_tensor(self, p_in_tensor, max_pool=False):
        if self.method_ == "poisson_disk":
            return torch.index_select(p_in_tensor, 0, self.pooling_ids_)
        ids = self.pooling_ids_.to(torch.int64)
        index = ids.reshape(-1, *([1] * (p_in_tensor.dim() - 1))).expand_as(p_in_tensor)
        out = torch.zeros((self.num_pooling_pts_,) + tuple(p_in_tensor.shape[1:]), dtype=p_in_tensor.dtype,
                          device=p_in_tensor.device)
        reduce = "amax" if max_pool else "mean"
        return out.scatter_reduce(0, index, p_in_tensor, reduce=reduce, include_self=False)
