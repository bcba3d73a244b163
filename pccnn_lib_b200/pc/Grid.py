import math

import torch

from .. import ops
from ..op_wrappers import BuildGridDS, ComputeKeys


class Grid(object):
    """Distributes the points of a batch into a regular grid
    (pccnn_lib/pc/Grid.py:10-72 of the reference).

    ``num_cells_`` is shared by all clouds of the batch.  ``compute_cell_ids`` fills ``cell_ids_``
    (int64 key per point) and ``sorted_ids_`` (the STABLE ascending permutation; the reference's
    torch.argsort leaves the order of equal keys open).  ``build_ds`` fills ``grid_ds_``.
    The sort also leaves the keys and points in sorted order in ``sorted_cell_ids_`` /
    ``sorted_pts_`` so that Neighborhood and PointPooling need no further gathers.
    """

    def __init__(self, p_point_cloud, p_bounding_box, p_cell_size):
        self.pointcloud_ = p_point_cloud
        self.bounding_box_ = p_bounding_box
        self.cell_size_ = torch.as_tensor(p_cell_size, device=self.pointcloud_.pts_.device).to(torch.float32)
        if self.cell_size_.dim() == 0:
            self.cell_size_ = self.cell_size_.repeat(self.pointcloud_.pts_.shape[1])
        with torch.no_grad():
            self.num_cells_ = ops.grid_num_cells(self.bounding_box_.min_, self.bounding_box_.max_, self.cell_size_)
        self.cell_ids_ = None
        self.sorted_ids_ = None
        self.sorted_cell_ids_ = None
        self.sorted_pts_ = None
        self.grid_ds_ = None

    def compute_cell_ids(self):
        if self.cell_ids_ is None:
            with torch.no_grad():
                pts = self.pointcloud_.pts_.detach()
                self.cell_ids_ = ComputeKeys.apply(pts, self.pointcloud_.batch_ids_, self.bounding_box_.min_,
                                                   self.num_cells_, self.cell_size_)
                # keys are below batch * cells: sort only the bits that can be set
                cells = self.num_cells_.tolist()
                span = float(int(self.pointcloud_.batch_size_))
                for c in cells:
                    span *= c
                key_bits = min(64, max(1, int(math.ceil(math.log2(span + 1)))))
                self.sorted_cell_ids_, self.sorted_ids_, self.sorted_pts_ = ops.sort_keys(self.cell_ids_, key_bits, pts)

    def build_ds(self):
        if self.cell_ids_ is None or self.sorted_ids_ is None:
            raise RuntimeError('In order to build the data structure first the'
                               ' keys for each point has to be computed.')
        if self.grid_ds_ is None:
            with torch.no_grad():
                self.grid_ds_ = BuildGridDS.apply(self.sorted_cell_ids_, self.num_cells_,
                                                  self.pointcloud_.batch_size_)

    def __repr__(self):
        return "### Cell size:\n{}\n### Num cells:\n{}\n### Cell Ids:\n{}\n### Sorted Ids:\n{}\n### Grid Ds:\n{}".format(
            self.cell_size_, self.num_cells_, self.cell_ids_, self.sorted_ids_, self.grid_ds_)
