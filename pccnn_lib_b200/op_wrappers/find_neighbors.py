import torch

from .. import ops


class FindNeighbors(torch.autograd.Function):
    """Radius search on the grid (pccnn_lib/op_wrappers/find_neighbors.py:10-31 of the reference).
    Returns (neighbors [T, 2] int32, start_ids [M] int32 holding inclusive end offsets)."""

    @staticmethod
    def forward(ctx, p_pts, p_pt_keys, p_samples, p_sample_keys, p_grid_ds, p_grid_size, p_radius,
                p_max_neighbors):
        neighbors, start_ids = ops.find_neighbors(p_pts, p_pt_keys, p_samples, p_sample_keys, p_grid_ds,
                                                  p_grid_size, p_radius, p_max_neighbors)
        ctx.mark_non_differentiable(neighbors, start_ids)
        return neighbors, start_ids

    @staticmethod
    def backward(ctx, p_grads_neigh, p_grads_start_ids):
        return None, None, None, None, None, None, None, None
