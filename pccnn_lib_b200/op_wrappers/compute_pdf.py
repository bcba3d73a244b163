import torch

from .. import ops


class ComputePDF(torch.autograd.Function):
    """Kernel density estimate per point and its point gradient
    (pccnn_lib/op_wrappers/compute_pdf.py:10-57 of the reference)."""

    @staticmethod
    def forward(ctx, p_pts, p_neighbors, p_start_ids, p_bandwidth, p_manifold_dims):
        ctx.with_grads_ = p_pts.requires_grad
        if ctx.with_grads_:
            ctx.save_for_backward(p_pts, p_neighbors, p_start_ids, p_bandwidth)
            ctx.manifold_dims_ = p_manifold_dims
            # set by pc.Neighborhood on a list that is the uncapped neighborhood of the points in themselves
            ctx.full_self_ = bool(getattr(p_neighbors, "_pccnn_full_self", False))
        return ops.compute_pdf(p_manifold_dims, p_bandwidth, p_pts, p_neighbors, p_start_ids)

    @staticmethod
    def backward(ctx, p_grads):
        pt_grads = None
        if ctx.with_grads_:
            pts, neighbors, start_ids, bandwidth = ctx.saved_tensors
            pt_grads = ops.compute_pdf_grads(ctx.manifold_dims_, bandwidth, pts, neighbors, start_ids,
                                             p_grads.contiguous(), full_self_neighborhood=ctx.full_self_)
        return pt_grads, None, None, None, None
