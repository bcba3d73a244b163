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
        self.cell_ids_ = None
        self.sorted_ids_ = None
        self.sorted_cell_ids_ = None
        self.sorted_pts_ = None
        self.grid_ds_ = None
        self._num_cells_host = None
        self._grid_ds_ready = None
        with torch.no_grad():
            bb = self.bounding_box_
            if getattr(bb, "_min", 0) is None and getattr(bb, "point_cloud_", None) is self.pointcloud_:
                # The box has not been evaluated yet and belongs to the same points: box, cells per axis,
                # keys, sort and cell table in one fused call (one host synchronisation instead of three).
                pc = self.pointcloud_
                r = ops.grid_front_end(pc.pts_.detach(), pc.batch_ids_, pc.batch_size_host(), self.cell_size_)
                bb._min, bb._max = r["aabb_min"], r["aabb_max"]
                self.num_cells_ = r["num_cells"]
                self._num_cells_host = r["num_cells_host"]
                self._fused = r
            else:
                self._fused = None
                self.num_cells_ = ops.grid_num_cells(bb.min_, bb.max_, self.cell_size_)

    def compute_cell_ids(self):
        if self.cell_ids_ is None:
            with torch.no_grad():
                if self._fused is not None:
                    r = self._fused
                    self.cell_ids_, self.sorted_cell_ids_ = r["keys"], r["sorted_keys"]
                    self.sorted_ids_, self.sorted_pts_ = r["sorted_ids"], r["sorted_pts"]
                    self._grid_ds_ready = r["grid_ds"]
                    self._fused = None
                    return
                pts = self.pointcloud_.pts_.detach()
                self.cell_ids_ = ComputeKeys.apply(pts, self.pointcloud_.batch_ids_, self.bounding_box_.min_,
                                                   self.num_cells_, self.cell_size_)
                # keys are below batch * cells: sort only the bits that can be set
                self._num_cells_host = self.num_cells_.tolist()
                span = float(self.pointcloud_.batch_size_host())
                for c in self._num_cells_host:
                    span *= c
                key_bits = min(64, max(1, int(math.ceil(math.log2(span + 1)))))
                self.sorted_cell_ids_, self.sorted_ids_, self.sorted_pts_ = ops.sort_keys(self.cell_ids_, key_bits, pts)

    def key_bits(self):
        """Number of low bits a key of this grid can have set (0 when the cells per axis are not known on
        the host yet)."""
        if self._num_cells_host is None:
            return 0
        span = float(self.pointcloud_.batch_size_host())
        for c in self._num_cells_host:
            span *= c
        return min(64, max(1, int(math.ceil(math.log2(span + 1)))))

    def build_ds(self):
        if self.cell_ids_ is None or self.sorted_ids_ is None:
            raise RuntimeError('In order to build the data structure first the'
                               ' keys for each point has to be computed.')
        if self.grid_ds_ is None:
            if self._grid_ds_ready is not None:
                self.grid_ds_, self._grid_ds_ready = self._grid_ds_ready, None
                return
            with torch.no_grad():
                self.grid_ds_ = BuildGridDS.apply(self.sorted_cell_ids_, self.num_cells_,
                                                  self.pointcloud_.batch_size_host(), self._num_cells_host)

    def __repr__(self):
        return "### Cell size:\n{}\n### Num cells:\n{}\n### Cell Ids:\n{}\n### Sorted Ids:\n{}\n### Grid Ds:\n{}".format(
            self.cell_size_, self.num_cells_, self.cell_ids_, self.sorted_ids_, self.grid_ds_)
