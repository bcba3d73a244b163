"""GPU parity: keys, sort, cell table, neighbor lists, KDE and Poisson-disk selection computed
through the C ABI must equal the CPU oracle bit for bit (float results within the stated
tolerance), on the reference's own test cases and on seeded ragged clouds."""
import numpy as np
import pytest
import torch

from conftest import ref_case, synthetic_case
from gpu_helpers import assert_grid_equal, both_neighborhoods, dev, gpu_grid
from oracle import oracle

pytestmark = pytest.mark.gpu

GRID_CASES = [(16, 1000, 2, 0.2), (16, 1000, 3, 0.2), (16, 1000, 6, 0.2), (16, 100, 2, 1.0), (16, 100, 3, 1.0),
              (16, 100, 6, 1.0), (32, 1000, 3, 0.05), (4, 1000, 4, 0.1), (4, 1000, 5, 0.3)]


@pytest.mark.parametrize("batch_size,num_pts,num_dims,radius", GRID_CASES)
def test_grid_is_bit_exact_on_reference_cases(ref_clouds, batch_size, num_pts, num_dims, radius):
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    cell = np.full((num_dims,), radius, np.float32)
    assert_grid_equal(gpu_grid(pts, batch_ids, batch_size, cell), oracle.build_grid(pts, batch_ids, batch_size, cell))


@pytest.mark.parametrize("seed,batch_size,num_pts,num_dims,radius",
                         [(1, 3, 5000, 3, 0.07), (2, 5, 3000, 2, 0.03), (3, 2, 20000, 3, 0.11), (4, 7, 999, 4, 0.25),
                          (5, 1, 1, 3, 0.5), (6, 2, 40000, 3, 0.013)])
def test_grid_is_bit_exact_on_ragged_clouds(seed, batch_size, num_pts, num_dims, radius):
    pts, batch_ids = synthetic_case(seed, batch_size, num_pts, num_dims)
    cell = (np.full((num_dims,), radius) * np.linspace(1.0, 1.3, num_dims)).astype(np.float32)  # anisotropic
    assert_grid_equal(gpu_grid(pts, batch_ids, batch_size, cell), oracle.build_grid(pts, batch_ids, batch_size, cell))


NEIGH_CASES = [(16, 100, 2, 1.0, 0), (16, 100, 3, 1.0, 0), (16, 100, 6, 1.0, 0), (4, 1000, 2, 0.2, 0),
               (4, 1000, 3, 0.2, 0), (4, 1000, 6, 0.2, 0), (4, 1000, 2, 0.2, 4), (4, 1000, 3, 0.2, 4),
               (4, 1000, 6, 0.2, 4), (8, 1000, 3, 0.05, 0), (8, 1000, 3, 0.1, 300), (4, 1000, 4, 0.15, 7)]


@pytest.mark.parametrize("batch_size,num_pts,num_dims,radius,max_neighs", NEIGH_CASES)
def test_neighbor_lists_are_identical_on_reference_cases(ref_clouds, batch_size, num_pts, num_dims, radius, max_neighs):
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    gn, gs, on, os_, _, _ = both_neighborhoods(pts, batch_ids, batch_size, radius, max_neighs)
    assert np.array_equal(gs.cpu().numpy(), os_)
    assert np.array_equal(gn.cpu().numpy(), on)  # same rows in the same (ascending) order


def test_uncapped_neighbor_sets_equal_brute_force(ref_clouds):
    pts, batch_ids = ref_case(ref_clouds, 4, 1000, 3)
    gn, gs, _, _, g, _ = both_neighborhoods(pts, batch_ids, 4, 0.2, 0)
    gn, gs = gn.cpu().numpy(), gs.cpu().numpy()
    sids = g["sorted_ids"].cpu().numpy()
    brute = oracle.brute_force_neighbors(pts, batch_ids, pts, batch_ids, 0.2)
    for m in range(pts.shape[0]):
        lo = 0 if m == 0 else gs[m - 1]
        assert np.array_equal(np.sort(sids[gn[lo:gs[m], 0]]), brute[m])


@pytest.mark.parametrize("seed,batch_size,num_pts,num_dims,radius,max_neighs",
                         [(11, 3, 4000, 3, 0.09, 0), (12, 4, 3000, 2, 0.05, 0), (13, 2, 2500, 5, 0.4, 0),
                          (14, 3, 4000, 3, 0.12, 16), (15, 1, 20000, 3, 0.05, 0)])
def test_neighbor_lists_with_separate_samples(seed, batch_size, num_pts, num_dims, radius, max_neighs):
    # samples are a different, unsorted point set; some fall outside the clouds' bounding boxes
    pts, batch_ids = synthetic_case(seed, batch_size, num_pts, num_dims)
    rs = np.random.RandomState(seed + 100)
    pick = rs.permutation(pts.shape[0])[: pts.shape[0] // 3]
    samples = (pts[pick] + rs.normal(0, radius * 0.5, size=(len(pick), num_dims))).astype(np.float32)
    gn, gs, on, os_, _, _ = both_neighborhoods(pts, batch_ids, batch_size, radius, max_neighs, samples, batch_ids[pick])
    assert np.array_equal(gs.cpu().numpy(), os_)
    assert np.array_equal(gn.cpu().numpy(), on)


def test_points_at_the_radius_boundary():
    # Pairs placed within a few ulps of the radius: the float operation order decides.
    rs = np.random.RandomState(7)
    r = np.float32(0.1)
    base = rs.rand(2000, 3).astype(np.float32)
    dirs = rs.normal(size=(2000, 3))
    dirs /= np.linalg.norm(dirs, axis=1, keepdims=True)
    scale = (1.0 + rs.randint(-4, 5, size=(2000, 1)) * 6e-8)
    other = (base.astype(np.float64) + dirs * float(r) * scale).astype(np.float32)
    pts = np.concatenate([base, other], 0)
    batch_ids = np.zeros(pts.shape[0], np.int32)
    gn, gs, on, os_, _, _ = both_neighborhoods(pts, batch_ids, 1, float(r), 0)
    assert np.array_equal(gs.cpu().numpy(), os_)
    assert np.array_equal(gn.cpu().numpy(), on)


def test_empty_inputs():
    from pccnn_lib_b200 import ops
    pts, batch_ids = synthetic_case(3, 2, 500, 3)
    cell = np.full((3,), 0.2, np.float32)
    g = gpu_grid(pts, batch_ids, 2, cell)
    empty_s = torch.zeros((0, 3), dtype=torch.float32, device="cuda")
    empty_k = torch.zeros((0,), dtype=torch.int64, device="cuda")
    n, s = ops.find_neighbors(g["sorted_pts"], g["sorted_keys"], empty_s, empty_k, g["grid_ds"], g["num_cells"],
                              g["cell"], 0)
    assert tuple(n.shape) == (0, 2) and tuple(s.shape) == (0,)
    # samples far away from every point: all segments empty
    far = dev(np.full((5, 3), 1e3, np.float32))
    fk = ops.compute_keys(far, dev(np.zeros(5, np.int32)), g["aabb_min"], g["num_cells"], g["cell"])
    n, s = ops.find_neighbors(g["sorted_pts"], g["sorted_keys"], far, fk, g["grid_ds"], g["num_cells"], g["cell"], 0)
    assert n.shape[0] == 0 and s.cpu().tolist() == [0] * 5
    assert ops.compute_keys(empty_s, torch.zeros((0,), dtype=torch.int32, device="cuda"), g["aabb_min"],
                            g["num_cells"], g["cell"]).shape[0] == 0
    # the list-free sampling of an empty set selects nothing; the fused front end refuses it (no bounding box)
    sel = ops.poisson_disk_sampling_grid(empty_s, empty_k, g["grid_ds"], g["num_cells"], g["cell"])
    assert tuple(sel.shape) == (0, 1)
    with pytest.raises(RuntimeError):
        ops.grid_front_end(empty_s, torch.zeros((0,), dtype=torch.int32, device="cuda"), 2, g["cell"])
    # a cloud of the batch without any point: same tables as the operator-by-operator path
    one_cloud = batch_ids == 0
    r = ops.grid_front_end(dev(pts[one_cloud]), dev(np.zeros(int(one_cloud.sum()), np.int32)), 1, g["cell"])
    o1 = oracle.build_grid(pts[one_cloud], np.zeros(int(one_cloud.sum()), np.int32), 1, cell)
    assert np.array_equal(r["sorted_ids"].cpu().numpy(), o1["sorted_ids"]) and np.array_equal(r["grid_ds"].cpu().numpy(), o1["grid_ds"])


PDF_CASES = [(4, 1000, 2, 0.02), (4, 1000, 3, 0.01), (4, 1000, 6, 0.01), (4, 1000, 2, 0.025), (4, 1000, 3, 0.025),
             (4, 1000, 6, 0.025), (8, 1000, 3, 0.05)]


@pytest.mark.parametrize("batch_size,num_pts,num_dims,bandwidth", PDF_CASES)
def test_pdf_and_grads_match_oracle(ref_clouds, batch_size, num_pts, num_dims, bandwidth):
    from pccnn_lib_b200 import ops
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    radius = float(np.float32(bandwidth) * np.float32(4.0))
    gn, gs, on, os_, g, o = both_neighborhoods(pts, batch_ids, batch_size, radius, 300)
    assert np.array_equal(gn.cpu().numpy(), on)
    bw = np.full((num_dims,), bandwidth, np.float32)
    # the op is fed the sorted points with rows indexing them (sample m = original point m)
    spts = o["sorted_pts"]
    # neighbors index sorted points but samples are the original order: build lists in one index space
    gn2, gs2, on2, os2, g2, o2 = both_neighborhoods(spts, batch_ids[o["sorted_ids"]], batch_size, radius, 300)
    got = ops.compute_pdf(num_dims, dev(bw), dev(spts), gn2, gs2).cpu().numpy()
    expect = oracle.compute_pdf(num_dims, bw, spts, on2, os2)
    # float32 sums in a different order: relative 1e-5 (typical error is ~1e-7 per term)
    assert np.allclose(got, expect, rtol=1e-5, atol=0)
    w = np.random.RandomState(5).randn(spts.shape[0]).astype(np.float32)
    gg = ops.compute_pdf_grads(num_dims, dev(bw), dev(spts), gn2, gs2, dev(w)).cpu().numpy()
    eg = oracle.compute_pdf_grads(num_dims, bw, spts, on2, os2, w)
    scale = np.abs(eg).max() + 1e-30
    assert np.abs(gg - eg).max() <= 2e-5 * scale  # float atomics vs a double-precision sum


@pytest.mark.parametrize("batch_size,num_pts,num_dims,bandwidth", PDF_CASES)
def test_pdf_grads_on_the_full_self_neighborhood(ref_clouds, batch_size, num_pts, num_dims, bandwidth):
    # The uncapped neighborhood of the points in themselves holds every pair in both rows; the one-pass gradient
    # for such lists against the oracle's general double-precision sum and against the general kernel.
    from pccnn_lib_b200 import ops
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    radius = float(np.float32(bandwidth) * np.float32(4.0))
    _, _, _, _, _, o = both_neighborhoods(pts, batch_ids, batch_size, radius, 0)
    spts = o["sorted_pts"]
    gn, gs, on, os_, _, _ = both_neighborhoods(spts, batch_ids[o["sorted_ids"]], batch_size, radius, 0)
    rows = gn.cpu().numpy()
    assert {(int(a), int(b)) for a, b in rows} == {(int(b), int(a)) for a, b in rows}  # the premise
    bw = np.full((num_dims,), bandwidth, np.float32)
    w = np.random.RandomState(6).randn(spts.shape[0]).astype(np.float32)
    one_pass = ops.compute_pdf_grads(num_dims, dev(bw), dev(spts), gn, gs, dev(w), full_self_neighborhood=True).cpu().numpy()
    general = ops.compute_pdf_grads(num_dims, dev(bw), dev(spts), gn, gs, dev(w)).cpu().numpy()
    expect = oracle.compute_pdf_grads(num_dims, bw, spts, on, os_, w)
    scale = np.abs(expect).max() + 1e-30
    assert np.abs(one_pass - expect).max() <= 2e-5 * scale
    assert np.abs(one_pass - general).max() <= 2e-5 * scale


PDS_CASES = [(4, 1000, 2, 0.1), (4, 1000, 3, 0.1), (4, 1000, 6, 0.1), (32, 100, 2, 3.0), (32, 100, 3, 3.0),
             (21, 100, 6, 3.0), (16, 1000, 3, 0.03), (8, 1000, 3, 0.3),
             # crowded cells (block per cell), cells beyond the block kernel's 512 points, thinned (one-sided) lists
             (4, 1000, 3, 0.5), (3, 1000, 2, 0.4), (2, 1000, 3, 1.0), (2, 1000, 4, 0.7),
             (4, 1000, 3, 0.5, 8), (8, 1000, 3, 0.3, 5), (2, 1000, 3, 1.0, 40)]


@pytest.mark.parametrize("case", PDS_CASES, ids=lambda c: "-".join(str(v) for v in c))
def test_poisson_disk_selection_is_identical(ref_clouds, case):
    batch_size, num_pts, num_dims, radius = case[:4]
    max_neighs = case[4] if len(case) > 4 else 0
    from pccnn_lib_b200 import ops
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    cell = np.full((num_dims,), radius, np.float32)
    g = gpu_grid(pts, batch_ids, batch_size, cell)
    o = oracle.build_grid(pts, batch_ids, batch_size, cell)
    gn, gs = ops.find_neighbors(g["sorted_pts"], g["sorted_keys"], g["sorted_pts"], g["sorted_keys"], g["grid_ds"],
                                g["num_cells"], g["cell"], max_neighs)
    # the oracle's thinning keeps other rows than the library's: both selections run on the library's lists
    on, os_ = gn.cpu().numpy(), gs.cpu().numpy()
    if max_neighs == 0:
        on0, os0 = oracle.find_neighbors(o["sorted_pts"], o["sorted_keys"], o["sorted_pts"], o["sorted_keys"],
                                         o["grid_ds"], o["num_cells"], cell, 0)
        assert np.array_equal(on, on0) and np.array_equal(os_, os0)
    got = ops.poisson_disk_sampling(g["sorted_keys"], gn, gs, g["num_cells"])
    expect = oracle.poisson_disk_sampling(o["sorted_keys"], on, os_, o["num_cells"])
    assert got.dtype == torch.int64 and got.dim() == 2 and got.shape[1] == 1
    assert np.array_equal(got.cpu().numpy(), expect)


@pytest.mark.parametrize("scratch", ["minimum", "partial"])
@pytest.mark.parametrize("max_neighs", [0, 16])
def test_neighbor_lists_do_not_depend_on_the_scratch_size(ref_clouds, scratch, max_neighs):
    # With little scratch the store pass repeats the distance tests instead of replaying the
    # bits kept by the count pass; with some scratch both paths run in one call.
    from pccnn_lib_b200 import _capi, ops
    pts, batch_ids = ref_case(ref_clouds, 16, 1000, 3)
    cell = np.full((3,), 0.15, np.float32)
    g = gpu_grid(pts, batch_ids, 16, cell)
    args = (g["sorted_pts"], g["sorted_keys"], g["sorted_pts"], g["sorted_keys"], g["grid_ds"], g["num_cells"],
            g["cell"], max_neighs)
    full_n, full_s = ops.find_neighbors(*args)
    lo = _capi.lib.pccnn_find_neighbors_min_workspace_bytes(3, pts.shape[0])
    nbytes = lo if scratch == "minimum" else lo + 40000
    n, s = ops.find_neighbors(*args, workspace_bytes=nbytes)
    assert torch.equal(s, full_s) and torch.equal(n, full_n)


@pytest.mark.parametrize("case", PDS_CASES[:12], ids=lambda c: "-".join(str(v) for v in c))
def test_grid_based_poisson_disk_sampling_makes_the_same_selection(ref_clouds, case):
    # No neighbor list: same passes and order, selected points kept per cell.  Must equal the list-based
    # operator (and the oracle) on the full radius-neighborhood.
    from pccnn_lib_b200 import ops
    batch_size, num_pts, num_dims, radius = case[:4]
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    cell = np.full((num_dims,), radius, np.float32)
    g = gpu_grid(pts, batch_ids, batch_size, cell)
    o = oracle.build_grid(pts, batch_ids, batch_size, cell)
    on, os_ = oracle.find_neighbors(o["sorted_pts"], o["sorted_keys"], o["sorted_pts"], o["sorted_keys"], o["grid_ds"],
                                    o["num_cells"], cell, 0)
    expect = oracle.poisson_disk_sampling(o["sorted_keys"], on, os_, o["num_cells"])
    got = ops.poisson_disk_sampling_grid(g["sorted_pts"], g["sorted_keys"], g["grid_ds"], g["num_cells"], g["cell"])
    assert got.dtype == torch.int64 and got.dim() == 2 and got.shape[1] == 1
    assert np.array_equal(got.cpu().numpy(), expect)


@pytest.mark.parametrize("seed,batch,num_pts,dims,radius", [(41, 6, 30000, 3, 0.05), (42, 3, 20000, 2, 0.02),
                                                            (43, 4, 40000, 3, 0.3), (44, 2, 3000, 5, 0.5)])
def test_grid_based_and_list_based_sampling_agree_on_larger_ragged_batches(seed, batch, num_pts, dims, radius):
    # thousands of cells per pass, sparse and crowded cells side by side; both operators on the GPU
    from conftest import synthetic_case
    from pccnn_lib_b200 import ops
    pts, batch_ids = synthetic_case(seed, batch, num_pts, dims)
    cell = np.full((dims,), radius, np.float32)
    g = gpu_grid(pts, batch_ids, batch, cell)
    nb, st = ops.find_neighbors(g["sorted_pts"], g["sorted_keys"], g["sorted_pts"], g["sorted_keys"], g["grid_ds"],
                                g["num_cells"], g["cell"], 0)
    by_list = ops.poisson_disk_sampling(g["sorted_keys"], nb, st, g["num_cells"])
    by_grid = ops.poisson_disk_sampling_grid(g["sorted_pts"], g["sorted_keys"], g["grid_ds"], g["num_cells"], g["cell"])
    assert by_list.shape[0] > 0 and torch.equal(by_list, by_grid)


def test_pdf_with_and_without_the_optional_scratch_is_bitwise_the_same(ref_clouds):
    # 3-D: with scratch the neighbors are gathered from a padded copy of the points; same terms, same order
    import ctypes
    from pccnn_lib_b200 import _capi, ops
    pts, batch_ids = ref_case(ref_clouds, 4, 1000, 3)
    gn, gs, on, os_, g, o = both_neighborhoods(pts, batch_ids, 4, 0.1, 0)
    spts = dev(o["sorted_pts"])
    bw = dev(np.full((3,), 0.025, np.float32))
    with_scratch = ops.compute_pdf(3, bw, spts, gn, gs)
    plain = torch.empty_like(with_scratch)
    rc = _capi.lib.pccnn_compute_pdf(3, 3, bw.data_ptr(), spts.shape[0], spts.data_ptr(), gn.data_ptr(), gs.data_ptr(),
                                     plain.data_ptr(), None, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(with_scratch, plain)
