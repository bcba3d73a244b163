import torch

from .. import ops


class BuildGridDS(torch.autograd.Function):
    """Cell-range table [batch, cells0, cells1, 2] over sorted keys
    (pccnn_lib/op_wrappers/build_grid_ds_funct.py:10-23 of the reference).  The output shape is
    read back from the device tensors here, exactly as the reference wrapper does, unless the caller
    already holds the cells per axis on the host (optional fourth argument)."""

    @staticmethod
    def forward(ctx, p_keys, p_grid_size, p_batch_size, p_grid_size_host=None):
        batch = p_batch_size.tolist() if torch.is_tensor(p_batch_size) else int(p_batch_size)
        cells = p_grid_size[0:2].tolist() if p_grid_size_host is None else [int(v) for v in p_grid_size_host[0:2]]
        return ops.build_grid_ds(p_keys, p_grid_size, [batch] + cells + [2])

    @staticmethod
    def backward(ctx, p_grads):
        return None, None, None, None
