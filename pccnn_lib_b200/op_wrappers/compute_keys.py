import torch

from .. import ops


class ComputeKeys(torch.autograd.Function):
    """Grid key of every point (pccnn_lib/op_wrappers/compute_keys.py:10-25 of the reference).
    Integer output: no gradient flows to any input."""

    @staticmethod
    def forward(ctx, p_pts, p_batch_ids, p_aabb_min, p_grid_size, p_cell_size):
        return ops.compute_keys(p_pts, p_batch_ids, p_aabb_min, p_grid_size, p_cell_size)

    @staticmethod
    def backward(ctx, p_grads):
        return None, None, None, None, None
