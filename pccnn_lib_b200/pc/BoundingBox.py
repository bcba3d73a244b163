from .. import ops


class BoundingBox(object):
    """Axis-aligned bounding box of every cloud of a batch, grown by 1e-6 on both sides
    (pccnn_lib/pc/BoundingBox.py:10-18 of the reference, which uses torch_scatter for it).

    Attributes: ``min_`` and ``max_``, float32 tensors [batch, dims].  They are computed on first
    use: a Grid built on the box right away computes them together with its keys in one fused call.
    """

    def __init__(self, p_point_cloud):
        self.point_cloud_ = p_point_cloud
        self._min = None
        self._max = None

    def _compute(self):
        pc = self.point_cloud_
        self._min, self._max = ops.bounding_box(pc.pts_.detach(), pc.batch_ids_, pc.batch_size_host())

    @property
    def min_(self):
        if self._min is None:
            self._compute()
        return self._min

    @property
    def max_(self):
        if self._max is None:
            self._compute()
        return self._max

    def __repr__(self):
        return "### Min:\n{}\n### Max:\n{}".format(self.min_, self.max_)
