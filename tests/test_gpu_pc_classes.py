"""The mirrored geometry classes (Pointcloud, BoundingBox, Grid, Neighborhood, PointPooling) driven
like the reference's tests drive them, compared with the oracle pipelines of test_oracle_pins."""
import numpy as np
import pytest
import torch

from conftest import ref_case
from test_oracle_pins import oracle_neighborhood, oracle_pdf, oracle_pooling

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch_size,num_pts,num_dims,radius,max_neighs",
                         [(16, 100, 3, 1.0, 0), (4, 1000, 2, 0.2, 0), (4, 1000, 3, 0.2, 4), (4, 1000, 6, 0.2, 0)])
def test_neighborhood_class_matches_oracle(ref_clouds, batch_size, num_pts, num_dims, radius, max_neighs):
    import pccnn_lib_b200 as lib
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    device = torch.device("cuda:0")
    pc = lib.pc.Pointcloud(pts, batch_ids, device=device)
    cell = np.full((num_dims,), radius, np.float32)
    bb = lib.pc.BoundingBox(pc)
    grid = lib.pc.Grid(pc, bb, cell)
    grid.compute_cell_ids()
    grid.build_ds()
    neigh = lib.pc.Neighborhood(grid, pc, max_neighs)
    expect_n, expect_s, g = oracle_neighborhood(pts, batch_ids, batch_size, radius, max_neighs)
    assert np.array_equal(grid.cell_ids_.cpu().numpy(), g["keys"])
    assert np.array_equal(grid.sorted_ids_.cpu().numpy(), g["sorted_ids"])
    assert np.array_equal(grid.grid_ds_.cpu().numpy(), g["grid_ds"])
    assert neigh.neighbors_.dtype == torch.int32 and neigh.start_ids_.dtype == torch.int32
    assert np.array_equal(neigh.start_ids_.cpu().numpy(), expect_s)
    assert np.array_equal(neigh.neighbors_.cpu().numpy(), expect_n)


@pytest.mark.parametrize("batch_size,num_pts,num_dims,radius", [(4, 1000, 2, 0.1), (4, 1000, 3, 0.1), (21, 100, 6, 3.0)])
def test_point_pooling_class_matches_oracle(ref_clouds, batch_size, num_pts, num_dims, radius):
    import pccnn_lib_b200 as lib
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    pc = lib.pc.Pointcloud(pts, batch_ids, device=torch.device("cuda:0"))
    pool = lib.pc.PointPooling(pc, np.full((num_dims,), radius, np.float32))
    expect = oracle_pooling(pts, batch_ids, batch_size, radius)
    assert pool.pooling_ids_.dtype == torch.int64
    assert np.array_equal(pool.pooling_ids_.cpu().numpy(), expect)
    pooled = pool.pool_tensor(pc.pts_)
    assert np.array_equal(pooled.cpu().numpy(), pts[expect])
    # cell_average mode is torch-only in the reference; check it against a NumPy mean per cell
    avg = lib.pc.PointPooling(pc, np.full((num_dims,), radius, np.float32), "cell_average")
    got = avg.pool_tensor(pc.pts_).cpu().numpy()
    ids = avg.pooling_ids_.cpu().numpy()
    want = np.stack([pts[ids == c].mean(0) for c in range(avg.num_pooling_pts_)])
    assert np.allclose(got, want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("batch_size,num_pts,num_dims,bandwidth", [(4, 1000, 2, 0.02), (4, 1000, 3, 0.025)])
def test_pointcloud_pdf_matches_oracle_and_backpropagates(ref_clouds, batch_size, num_pts, num_dims, bandwidth):
    import pccnn_lib_b200 as lib
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    pc = lib.pc.Pointcloud(pts, batch_ids, device=torch.device("cuda:0"), requires_grad=True)
    pc.compute_pdf(np.full((num_dims,), bandwidth, np.float32))
    expect, unnorm, _, _ = oracle_pdf(pts, batch_ids, batch_size, bandwidth)
    assert np.allclose(pc.pts_pdf_.detach().cpu().numpy(), expect, rtol=1e-5, atol=0)
    assert np.allclose(pc.pts_unnorm_pdf_.detach().cpu().numpy(), unnorm, rtol=1e-5, atol=0)
    pc.pts_pdf_.mean().backward()
    assert pc.pts_.grad is not None and torch.isfinite(pc.pts_.grad).all() and pc.pts_.grad.abs().sum() > 0
    assert tuple(pc.global_pooling(pc.pts_.detach(), "max").shape) == (batch_size, num_dims)


def test_density_gradient_through_the_classes_uses_the_full_self_neighborhood(ref_clouds):
    # Neighborhood marks the uncapped neighborhood of a cloud in itself; ComputePDF hands the mark to the gradient
    # operator.  Same gradient as with the mark removed (general kernel).
    import pccnn_lib_b200 as lib
    from pccnn_lib_b200.op_wrappers import ComputePDF
    pts, batch_ids = ref_case(ref_clouds, 4, 800, 3)
    bw = torch.full((3,), 0.03, dtype=torch.float32, device="cuda:0")
    grads = []
    for keep_mark in (True, False):
        pc = lib.pc.Pointcloud(torch.as_tensor(pts, device="cuda:0").requires_grad_(True),
                               torch.as_tensor(batch_ids, device="cuda:0"))
        grid = lib.pc.Grid(pc, lib.pc.BoundingBox(pc), bw * 4.0)
        grid.compute_cell_ids()
        grid.build_ds()
        nb = lib.pc.Neighborhood(grid, pc, 0)
        assert nb.full_self_ and nb.neighbors_._pccnn_full_self
        capped = lib.pc.Neighborhood(grid, pc, 300)
        assert not capped.full_self_
        if not keep_mark:
            nb.neighbors_._pccnn_full_self = False
        pdf = ComputePDF.apply(pc.pts_, nb.neighbors_, nb.start_ids_, bw, 3)
        (pdf * torch.linspace(0.5, 1.5, pdf.shape[0], device="cuda:0")).sum().backward()
        grads.append(pc.pts_.grad.detach().cpu().numpy())
    assert np.abs(grads[0]).max() > 0
    assert np.abs(grads[0] - grads[1]).max() <= 2e-5 * np.abs(grads[1]).max()


def test_reference_module_names_resolve_to_this_package():
    import sys
    import pccnn_lib_b200
    pccnn_lib_b200.install_as_reference_modules()
    import pccnn_lib_ops
    import pccnn_lib
    assert pccnn_lib_ops.compute_keys is pccnn_lib_b200.ops.compute_keys
    assert pccnn_lib.pc.KPConv is pccnn_lib_b200.pc.layers.KPConv
    for name in ("build_grid_ds", "compute_keys", "find_neighbors", "compute_pdf", "compute_pdf_grads",
                 "poisson_disk_sampling", "kp_conv", "kp_conv_grads", "mc_conv", "mc_conv_grads"):
        assert callable(getattr(pccnn_lib_ops, name))
    for m in ("pccnn_lib_ops", "pccnn_lib", "pccnn_lib.pc", "pccnn_lib.op_wrappers"):
        sys.modules.pop(m, None)


@pytest.mark.parametrize("dims,cell", [(3, 0.1), (2, 0.25), (5, 0.6)])
def test_fused_grid_front_end_equals_the_separate_operators_and_the_oracle(ref_clouds, dims, cell):
    # One fused call (one host synchronisation) against the operator-by-operator sequence and the CPU oracle.
    from pccnn_lib_b200 import ops
    from oracle import oracle
    _t = lambda a: torch.as_tensor(a, device="cuda:0")
    pts, batch_ids = ref_case(ref_clouds, 6, 700, dims)
    cell_size = np.full((dims,), cell, np.float32)
    r = ops.grid_front_end(_t(pts), _t(batch_ids), 6, _t(cell_size))
    o = oracle.build_grid(pts, batch_ids, 6, cell_size)
    assert r["num_cells_host"] == list(o["num_cells"])
    for mine, ref in (("aabb_min", "aabb_min"), ("aabb_max", "aabb_max"), ("num_cells", "num_cells"), ("keys", "keys"),
                      ("sorted_keys", "sorted_keys"), ("sorted_ids", "sorted_ids"), ("sorted_pts", "sorted_pts"),
                      ("grid_ds", "grid_ds")):
        assert np.array_equal(r[mine].cpu().numpy(), np.asarray(o[ref])), mine


def test_grid_on_an_unevaluated_box_takes_the_fused_path_with_equal_results(ref_clouds):
    import pccnn_lib_b200 as lib
    _t = lambda a: torch.as_tensor(a, device="cuda:0")
    pts, batch_ids = ref_case(ref_clouds, 5, 600, 3)
    cell_size = np.full((3,), 0.15, np.float32)
    pc = lib.pc.Pointcloud(_t(pts), _t(batch_ids))
    fused = lib.pc.Grid(pc, lib.pc.BoundingBox(pc), cell_size)           # box not touched before: fused call
    assert fused._fused is not None
    box = lib.pc.BoundingBox(pc)
    box.min_                                                             # evaluated: operator-by-operator path
    plain = lib.pc.Grid(pc, box, cell_size)
    assert plain._fused is None
    for g in (fused, plain):
        g.compute_cell_ids()
        g.build_ds()
    for name in ("num_cells_", "cell_ids_", "sorted_ids_", "sorted_cell_ids_", "sorted_pts_", "grid_ds_"):
        assert torch.equal(getattr(fused, name), getattr(plain, name)), name
    assert torch.equal(fused.bounding_box_.min_, box.min_) and torch.equal(fused.bounding_box_.max_, box.max_)
