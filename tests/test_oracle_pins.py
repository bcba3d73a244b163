"""Pins the CPU oracle against the expectations the reference's own unit tests compute.

The reference stores no golden files: each of its tests recomputes the expected result with
NumPy / scikit-learn from the 32 clouds of unit_test/point_clouds and compares.  These tests
replay those expectations (restated here, each citing its source) on the same clouds and the
same (batch_size, num_pts, num_dims, radius) cases as unit_test/utest_*.ini, with the oracle in
the place of the reference's GPU result.
"""
import numpy as np
import pytest

from conftest import ref_case
from oracle import oracle

CELL_CASES = [(16, 1000, 2, 0.2), (16, 1000, 3, 0.2), (16, 1000, 6, 0.2),
              (16, 100, 2, 1.0), (16, 100, 3, 1.0), (16, 100, 6, 1.0)]


def numpy_cell_ids(pts, batch_ids, batch_size, num_pts, num_dims, cell_size, grid_size):
    """unit_test/test_cell_ids.py:51-65 of the reference."""
    sel = pts.reshape((-1, num_pts, num_dims))
    diff = sel - np.amin(sel, 1, keepdims=True)
    idx = np.floor(diff / cell_size.reshape((1, 1, num_dims))).astype(np.int32).reshape((-1, num_dims))
    idx = np.maximum(np.zeros((1, num_dims), np.int32), np.minimum(idx, grid_size.reshape((1, num_dims))))
    ids = idx[:, -1].astype(np.int64)
    acc = int(grid_size[-1])
    for d in range(num_dims - 2, -1, -1):
        ids = ids + idx[:, d].astype(np.int64) * acc
        acc = acc * int(grid_size[d])
    return ids + batch_ids.astype(np.int64) * acc, acc


@pytest.mark.parametrize("batch_size,num_pts,num_dims,radius", CELL_CASES)
def test_bounding_box_matches_numpy(ref_clouds, batch_size, num_pts, num_dims, radius):
    # unit_test/test_bb.py:45-53: np.amin / np.amax per cloud, isclose 1e-5.
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    mn, mx = oracle.bounding_box(pts, batch_ids, batch_size)
    sel = pts.reshape((batch_size, num_pts, num_dims))
    assert np.allclose(mn, sel.min(1), atol=1e-5, rtol=0)
    assert np.allclose(mx, sel.max(1), atol=1e-5, rtol=0)
    assert np.array_equal(mn, sel.min(1) - np.float32(1e-6))
    assert np.array_equal(mx, sel.max(1) + np.float32(1e-6))


@pytest.mark.parametrize("batch_size,num_pts,num_dims,radius", CELL_CASES)
def test_cell_ids_match_reference_numpy(ref_clouds, batch_size, num_pts, num_dims, radius):
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    cell = np.full((num_dims,), radius, np.float32)
    g = oracle.build_grid(pts, batch_ids, batch_size, cell)
    expect, _ = numpy_cell_ids(pts, batch_ids, batch_size, num_pts, num_dims, cell, g["num_cells"])
    assert np.array_equal(g["keys"], expect)


@pytest.mark.parametrize("batch_size,num_pts,num_dims,radius", CELL_CASES)
def test_grid_ds_matches_reference_numpy(ref_clouds, batch_size, num_pts, num_dims, radius):
    # unit_test/test_grid_ds.py:69-98: walk the sorted ids and record first / one-past-last.
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    cell = np.full((num_dims,), radius, np.float32)
    g = oracle.build_grid(pts, batch_ids, batch_size, cell)
    gs = g["num_cells"]
    ids, acc = numpy_cell_ids(pts, batch_ids, batch_size, num_pts, num_dims, cell, gs)
    sorted_ids = ids[np.argsort(ids, kind="stable")]
    ds = np.zeros((batch_size, gs[0], gs[1], 2), np.int32)
    f0 = acc
    f1 = f0 // int(gs[0])
    f2 = f1 // int(gs[1])
    for it, cid in enumerate(sorted_ids):
        if it > 0:
            prev = sorted_ids[it - 1]
            if prev // f2 != cid // f2:
                ds[cid // f0, (cid // f1) % gs[0], (cid // f2) % gs[1], 0] = it
                ds[prev // f0, (prev // f1) % gs[0], (prev // f2) % gs[1], 1] = it
    last = sorted_ids[-1]
    ds[last // f0, (last // f1) % gs[0], (last // f2) % gs[1], 1] = len(sorted_ids)
    assert np.array_equal(g["grid_ds"], ds)


NEIGH_CASES = [(16, 100, 2, 1.0, 0), (16, 100, 3, 1.0, 0), (16, 100, 6, 1.0, 0),
               (4, 1000, 2, 0.2, 0), (4, 1000, 3, 0.2, 0), (4, 1000, 6, 0.2, 0),
               (4, 1000, 2, 0.2, 4), (4, 1000, 3, 0.2, 4), (4, 1000, 6, 0.2, 4)]


def oracle_neighborhood(pts, batch_ids, batch_size, radius, max_neighbors, samples=None, sample_batch_ids=None):
    """pccnn_lib/pc/Neighborhood.py:27-53 of the reference on top of the oracle: neighbor rows
    are mapped back to original point indices."""
    cell = np.full((pts.shape[1],), radius, np.float32)
    g = oracle.build_grid(pts, batch_ids, batch_size, cell)
    if samples is None:
        samples, sample_batch_ids = pts, batch_ids
    skeys = oracle.compute_keys(samples, sample_batch_ids, g["aabb_min"], g["num_cells"], cell)
    neigh, start_ids = oracle.find_neighbors(g["sorted_pts"], g["sorted_keys"], samples, skeys, g["grid_ds"],
                                             g["num_cells"], cell, max_neighbors)
    neigh = neigh.copy()
    neigh[:, 0] = g["sorted_ids"][neigh[:, 0]].astype(np.int32)
    return neigh, start_ids, g


@pytest.mark.parametrize("batch_size,num_pts,num_dims,radius,max_neighs", NEIGH_CASES)
def test_neighbors_match_reference_brute_force(ref_clouds, batch_size, num_pts, num_dims, radius, max_neighs):
    # unit_test/test_find_neighs.py:55-94: per sample, equal counts (or == max when capped) and
    # every listed neighbor is a brute-force neighbor.  Without a cap the sets must be equal.
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    neigh, start_ids, _ = oracle_neighborhood(pts, batch_ids, batch_size, radius, max_neighs)
    brute = oracle.brute_force_neighbors(pts, batch_ids, pts, batch_ids, radius)
    assert start_ids.shape[0] == pts.shape[0]
    for m in range(pts.shape[0]):
        lo = 0 if m == 0 else start_ids[m - 1]
        got = neigh[lo:start_ids[m]]
        assert np.all(got[:, 1] == m)
        if max_neighs > 0 and len(brute[m]) > max_neighs:
            assert len(got) == max_neighs
            assert len(np.unique(got[:, 0])) == max_neighs
            assert np.all(np.isin(got[:, 0], brute[m]))
        else:
            assert np.array_equal(np.sort(got[:, 0]), brute[m])


PDF_CASES = [(4, 1000, 2, 0.02), (4, 1000, 3, 0.01), (4, 1000, 6, 0.01),
             (4, 1000, 2, 0.025), (4, 1000, 3, 0.025), (4, 1000, 6, 0.025)]


def oracle_pdf(pts, batch_ids, batch_size, bandwidth):
    """pccnn_lib/pc/Pointcloud.py:81-109 of the reference on top of the oracle."""
    d = pts.shape[1]
    bw = np.full((d,), bandwidth, np.float32)
    neigh, start_ids, _ = oracle_neighborhood(pts, batch_ids, batch_size, np.float32(bandwidth) * np.float32(4.0), 300)
    unnorm = oracle.compute_pdf(d, bw, pts, neigh, start_ids)
    counts = np.bincount(batch_ids, minlength=batch_size)
    return unnorm / counts[batch_ids].astype(np.float32), unnorm, neigh, start_ids


@pytest.mark.parametrize("batch_size,num_pts,num_dims,bandwidth", PDF_CASES)
def test_pdf_matches_sklearn(ref_clouds, batch_size, num_pts, num_dims, bandwidth):
    # unit_test/test_pdf.py:50-60: sklearn KernelDensity per cloud, isclose(rtol=atol=1e-2).
    from sklearn.neighbors import KernelDensity
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    pdf, _, _, _ = oracle_pdf(pts, batch_ids, batch_size, bandwidth)
    sel = pts.reshape((batch_size, num_pts, num_dims))
    expect = []
    for b in range(batch_size):
        kde = KernelDensity(bandwidth=bandwidth)
        kde.fit(sel[b])
        expect.append(np.exp(kde.score_samples(sel[b])))
    expect = np.concatenate(expect, 0)
    assert np.isclose(expect, pdf, rtol=1e-2, atol=1e-2).all()


@pytest.mark.parametrize("batch_size,num_pts,num_dims,bandwidth", [(2, 100, 2, 0.1), (2, 100, 3, 0.15), (2, 100, 6, 0.2)])
def test_pdf_grads_match_finite_differences(ref_clouds, batch_size, num_pts, num_dims, bandwidth):
    # unit_test/test_pdf_grads.py:55-58 gradchecks mean(pdf) in float32 with eps=1e-3 and 1e-2
    # tolerances; here the analytic gradient of the oracle is compared with central differences
    # of a float64 restatement of the same sum over the same (fixed) neighbor lists.
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    _, _, neigh, start_ids = oracle_pdf(pts, batch_ids, batch_size, bandwidth)
    bw = np.full((num_dims,), bandwidth, np.float32)
    w = np.random.RandomState(0).randn(pts.shape[0]).astype(np.float32)
    grads = oracle.compute_pdf_grads(num_dims, bw, pts, neigh, start_ids, w)

    ibw = (1.0 / bw).astype(np.float64)
    scale = np.prod(ibw) / (2.0 * 3.1415) ** (num_dims / 2.0)

    def loss(p):
        diff = (p[neigh[:, 0]] - p[neigh[:, 1]]) * ibw
        return np.sum(w[neigh[:, 1]].astype(np.float64) * scale * np.exp(-0.5 * np.sum(diff * diff, -1)))

    p0 = pts.astype(np.float64)
    rs = np.random.RandomState(1)
    for _ in range(24):
        i, d = rs.randint(pts.shape[0]), rs.randint(num_dims)
        h = 1e-5
        pp, pm = p0.copy(), p0.copy()
        pp[i, d] += h
        pm[i, d] -= h
        num = (loss(pp) - loss(pm)) / (2 * h)
        assert np.isclose(grads[i, d], num, rtol=1e-3, atol=1e-3 * max(1.0, abs(num)))


PDS_CASES = [(4, 1000, 2, 0.1), (4, 1000, 3, 0.1), (4, 1000, 6, 0.1), (32, 100, 2, 3.0), (32, 100, 3, 3.0), (21, 100, 6, 3.0)]


def oracle_pooling(pts, batch_ids, batch_size, radius):
    """pccnn_lib/pc/PointPooling.py:39-69 of the reference on top of the oracle."""
    cell = np.full((pts.shape[1],), radius, np.float32)
    g = oracle.build_grid(pts, batch_ids, batch_size, cell)
    neigh, start_ids = oracle.find_neighbors(g["sorted_pts"], g["sorted_keys"], g["sorted_pts"], g["sorted_keys"],
                                             g["grid_ds"], g["num_cells"], cell, 0)
    sel = oracle.poisson_disk_sampling(g["sorted_keys"], neigh, start_ids, g["num_cells"]).reshape(-1)
    return g["sorted_ids"][sel]


@pytest.mark.parametrize("batch_size,num_pts,num_dims,radius", PDS_CASES)
def test_pooling_has_reference_property(ref_clouds, batch_size, num_pts, num_dims, radius):
    # unit_test/test_pd_pooling.py:50-58: no two selected points of a cloud closer than the radius.
    # Added: maximality (every rejected point has a selected neighbor), which the reference
    # does not check.
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    ids = oracle_pooling(pts, batch_ids, batch_size, radius)
    sel_pts, sel_b = pts[ids], batch_ids[ids]
    assert len(np.unique(ids)) == len(ids) and len(ids) > 0
    for i in range(len(ids)):
        diff = sel_pts[i].reshape(1, -1) - sel_pts
        dist = np.sqrt(np.sum(diff * diff, -1))
        mask = np.logical_and(dist < radius, sel_b == sel_b[i])
        mask[i] = False
        assert not mask.any()
    chosen = np.zeros(pts.shape[0], bool)
    chosen[ids] = True
    brute = oracle.brute_force_neighbors(pts, batch_ids, pts, batch_ids, radius)
    for i in range(pts.shape[0]):
        assert chosen[brute[i]].any()
