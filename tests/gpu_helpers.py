"""Shared helpers of the GPU parity tests: run the same pipeline through the C ABI
(pccnn_lib_b200.ops) and through the CPU oracle."""
import numpy as np
import torch

from oracle import oracle


def dev(a):
    return torch.as_tensor(np.ascontiguousarray(a), device="cuda")


def gpu_grid(pts, batch_ids, batch_size, cell):
    """BoundingBox + Grid of the reference's caller side, on the GPU through ops."""
    from pccnn_lib_b200 import ops
    p, b, c = dev(pts), dev(batch_ids), dev(cell)
    mn, mx = ops.bounding_box(p, b, batch_size)
    nc = ops.grid_num_cells(mn, mx, c)
    keys = ops.compute_keys(p, b, mn, nc, c)
    skeys, sids, spts = ops.sort_keys(keys, 64, p)
    shape = [batch_size] + nc[0:2].tolist() + [2]
    ds = ops.build_grid_ds(skeys, nc, shape)
    return dict(pts=p, batch_ids=b, cell=c, aabb_min=mn, aabb_max=mx, num_cells=nc, keys=keys, sorted_keys=skeys,
                sorted_ids=sids, sorted_pts=spts, grid_ds=ds)


def assert_grid_equal(g, o):
    assert np.array_equal(g["aabb_min"].cpu().numpy(), o["aabb_min"])
    assert np.array_equal(g["aabb_max"].cpu().numpy(), o["aabb_max"])
    assert np.array_equal(g["num_cells"].cpu().numpy(), o["num_cells"])
    assert np.array_equal(g["keys"].cpu().numpy(), o["keys"])
    assert np.array_equal(g["sorted_ids"].cpu().numpy(), o["sorted_ids"])
    assert np.array_equal(g["sorted_keys"].cpu().numpy(), o["sorted_keys"])
    assert np.array_equal(g["sorted_pts"].cpu().numpy(), o["sorted_pts"])
    assert np.array_equal(g["grid_ds"].cpu().numpy(), o["grid_ds"])


def both_neighborhoods(pts, batch_ids, batch_size, radius, max_neighbors, samples=None, sample_batch_ids=None):
    """(gpu neighbors, gpu start_ids, oracle neighbors, oracle start_ids, gpu grid, oracle grid) with rows
    indexing the SORTED point array, as the op itself returns them."""
    from pccnn_lib_b200 import ops
    d = pts.shape[1]
    cell = np.full((d,), radius, np.float32)
    g = gpu_grid(pts, batch_ids, batch_size, cell)
    o = oracle.build_grid(pts, batch_ids, batch_size, cell)
    if samples is None:
        samples, sample_batch_ids = pts, batch_ids
    s, sb = dev(samples), dev(sample_batch_ids)
    skeys = ops.compute_keys(s, sb, g["aabb_min"], g["num_cells"], g["cell"])
    okeys = oracle.compute_keys(samples, sample_batch_ids, o["aabb_min"], o["num_cells"], cell)
    assert np.array_equal(skeys.cpu().numpy(), okeys)
    gn, gs = ops.find_neighbors(g["sorted_pts"], g["sorted_keys"], s, skeys, g["grid_ds"], g["num_cells"],
                                g["cell"], max_neighbors)
    on, os_ = oracle.find_neighbors(o["sorted_pts"], o["sorted_keys"], samples, okeys, o["grid_ds"], o["num_cells"],
                                    cell, max_neighbors)
    return gn, gs, on, os_, g, o
