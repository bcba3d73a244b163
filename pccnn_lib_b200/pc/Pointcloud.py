import torch

from ..op_wrappers import ComputePDF


class Pointcloud(object):
    """A batch of point clouds: coordinates ``pts_`` [n, d] and ``batch_ids_`` [n]
    (pccnn_lib/pc/Pointcloud.py:11-170 of the reference; torch_scatter replaced by torch ops)."""

    def __init__(self, p_pts, p_batch_ids, p_manifold_dims=None, **kwargs):
        self.dim_manifold_ = p_pts.shape[1] if p_manifold_dims is None else p_manifold_dims
        self.pts_with_grads_ = kwargs.pop('requires_grad', False)
        self.pts_ = torch.as_tensor(p_pts, **kwargs)
        self.batch_ids_ = torch.as_tensor(p_batch_ids, **kwargs)
        self.batch_size_ = torch.max(self.batch_ids_) + 1
        self._batch_size_host = None
        if self.pts_with_grads_:
            self.pts_.requires_grad = True
        self.pts_pdf_ = None
        self.pts_unnorm_pdf_ = None

    def batch_size_host(self):
        """Number of clouds as a Python int; read from the device once and remembered."""
        if self._batch_size_host is None:
            self._batch_size_host = int(self.batch_size_)
        return self._batch_size_host

    def to_device(self, p_device):
        self.pts_ = self.pts_.to(p_device)
        self.batch_ids_ = self.batch_ids_.to(p_device)
        self.batch_size_ = self.batch_size_.to(p_device)
        if self.pts_unnorm_pdf_ is not None:
            self.pts_unnorm_pdf_ = self.pts_unnorm_pdf_.to(p_device)
            self.pts_pdf_ = self.pts_pdf_.to(p_device)

    def get_num_points_per_batch(self):
        with torch.no_grad():
            return torch.bincount(self.batch_ids_.to(torch.int64), minlength=self.batch_size_host()).to(torch.int32)

    def compute_pdf(self, p_badnwidth):
        """KDE of every point with the given per-axis bandwidth; neighbors are searched within
        4 bandwidths and capped at 300 per point (pccnn_lib/pc/Pointcloud.py:81-109)."""
        from .BoundingBox import BoundingBox
        from .Grid import Grid
        from .Neighborhood import Neighborhood
        bandwidth = torch.as_tensor(p_badnwidth, device=self.pts_.device).to(torch.float32)
        radii = bandwidth * 4.0
        aabb = BoundingBox(self)
        grid = Grid(self, aabb, radii)
        grid.compute_cell_ids()
        grid.build_ds()
        neigh = Neighborhood(grid, self, 300)
        self.pts_unnorm_pdf_ = ComputePDF.apply(self.pts_, neigh.neighbors_, neigh.start_ids_, bandwidth,
                                                self.dim_manifold_)
        num_pts = torch.index_select(self.get_num_points_per_batch(), 0, self.batch_ids_.to(torch.int64))
        self.pts_pdf_ = self.pts_unnorm_pdf_ / num_pts.to(torch.float32)

    def _pool(self, p_in_tensor, reduce):
        ids = self.batch_ids_.to(torch.int64)
        index = ids.reshape(-1, *([1] * (p_in_tensor.dim() - 1))).expand_as(p_in_tensor)
        out = torch.zeros((self.batch_size_host(),) + tuple(p_in_tensor.shape[1:]), dtype=p_in_tensor.dtype,
                          device=p_in_tensor.device)
        return out.scatter_reduce(0, index, p_in_tensor, reduce=reduce, include_self=False)

    def global_pooling(self, p_in_tensor, p_pooling_method="avg"):
        reduce = {"max": "amax", "min": "amin", "avg": "mean", "sum": "sum"}[p_pooling_method]
        return self._pool(p_in_tensor, reduce)

    def global_upsample(self, p_in_tensor):
        return torch.index_select(p_in_tensor, 0, self.batch_ids_.to(torch.int64))

    def __repr__(self):
        return "### Points:\n{}\n### Batch Ids:\n{}\n### Batch Size:\n{}\n### Pdf:\n{}".format(
            self.pts_, self.batch_ids_, self.batch_size_, self.pts_pdf_)

    def __torch_function__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        args = [a.pts_ if hasattr(a, 'pts_') else a for a in args]
        return Pointcloud(func(*args, **kwargs), self.batch_ids_)
