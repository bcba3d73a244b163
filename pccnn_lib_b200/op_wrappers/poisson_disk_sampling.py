import torch

from .. import ops


class PoissonDiskSamlping(torch.autograd.Function):
    """Poisson-disk selection over sorted points; the class name keeps the reference's spelling
    (pccnn_lib/op_wrappers/poisson_disk_sampling.py:10-24 of the reference)."""

    @staticmethod
    def forward(ctx, p_sorted_keys, p_neighbors, p_start_ids, p_grid_size):
        out = ops.poisson_disk_sampling(p_sorted_keys, p_neighbors, p_start_ids, p_grid_size)
        ctx.mark_non_differentiable(out)
        return out

    @staticmethod
    def backward(ctx, p_grads):
        return None, None, None, None
