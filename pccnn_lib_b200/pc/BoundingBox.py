from .. import ops


class BoundingBox(object):
    """Axis-aligned bounding box of every cloud of a batch, grown by 1e-6 on both sides
    (pccnn_lib/pc/BoundingBox.py:10-18 of the reference, which uses torch_scatter for it).

    Attributes: ``min_`` and ``max_``, float32 tensors [batch, dims].
    """

    def __init__(self, p_point_cloud):
        self.min_, self.max_ = ops.bounding_box(p_point_cloud.pts_.detach(), p_point_cloud.batch_ids_,
                                                int(p_point_cloud.batch_size_))

    def __repr__(self):
        return "### Min:\n{}\n### Max:\n{}".format(self.min_, self.max_)
