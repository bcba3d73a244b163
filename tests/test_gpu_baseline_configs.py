"""GPU parity on the geometry, shapes and sizes of the benchmark configurations (the other GPU tests run on the
reference's fixture clouds and small uniform sets): the surface sampler incl. a single small primitive with
crowded cells, the exact single-layer KPConv configuration, convolutions with more samples than one internal
chunk (131 072) so that the chunked projection / tensor-core path is compared with the oracle, and a batch
processed in shards against the oracle's full-batch result."""
import numpy as np
import pytest
import torch

from bench import scene_cloud, surface_cloud
from gpu_helpers import assert_grid_equal, dev, gpu_grid
from oracle import conv_oracle, oracle

pytestmark = pytest.mark.gpu


def _surface_batch(spec):
    """spec: list of (cloud id of the benchmark's sampler, points)."""
    pts = np.concatenate([surface_cloud(cid, n) for cid, n in spec], 0)
    ids = np.concatenate([np.full((n,), b, np.int32) for b, (_, n) in enumerate(spec)])
    return pts, ids


# cloud 13 of the sampler is one small primitive: every cell of it is crowded (hundreds of points per cell at
# radius 0.05), which is where the int32 neighbor count of the full configuration comes from
SURFACE_SPEC = [(13, 30000), (0, 20000), (5, 25000)]


@pytest.mark.parametrize("max_neighbors", [0, 300])
def test_surface_clouds_search_kde_and_sampling(max_neighbors):
    from pccnn_lib_b200 import ops
    pts, ids = _surface_batch(SURFACE_SPEC)
    radius = 0.05
    cell = np.full((3,), radius, np.float32)
    g = gpu_grid(pts, ids, len(SURFACE_SPEC), cell)
    o = oracle.build_grid(pts, ids, len(SURFACE_SPEC), cell)
    assert_grid_equal(g, o)
    gn, gs = ops.find_neighbors(g["sorted_pts"], g["sorted_keys"], g["sorted_pts"], g["sorted_keys"], g["grid_ds"],
                                g["num_cells"], g["cell"], max_neighbors)
    on, os_ = oracle.find_neighbors(o["sorted_pts"], o["sorted_keys"], o["sorted_pts"], o["sorted_keys"], o["grid_ds"],
                                    o["num_cells"], cell, max_neighbors)
    assert np.array_equal(gs.cpu().numpy(), os_)
    assert np.array_equal(gn.cpu().numpy(), on)  # same rows in the same (ascending) order, thinned lists included
    counts = np.diff(np.concatenate([[0], os_]))
    if max_neighbors == 0:
        assert counts[ids[o["sorted_ids"]] == 0].mean() > 300  # the dense cloud really is dense
    else:
        assert counts.max() == max_neighbors
    bw = np.full((3,), 0.01, np.float32)
    pdf = ops.compute_pdf(3, dev(bw), g["sorted_pts"], gn, gs).cpu().numpy()
    opdf = oracle.compute_pdf(3, bw, o["sorted_pts"], on, os_)
    assert np.allclose(pdf, opdf, rtol=1e-5, atol=0)
    w = np.random.RandomState(2).normal(size=(pts.shape[0],)).astype(np.float32)
    pg = ops.compute_pdf_grads(3, dev(bw), g["sorted_pts"], gn, gs, dev(w)).cpu().numpy()
    opg = oracle.compute_pdf_grads(3, bw, o["sorted_pts"], on, os_, w)
    assert np.abs(pg - opg).max() <= 2e-5 * np.abs(opg).max()
    if max_neighbors == 0:
        sel = ops.poisson_disk_sampling(g["sorted_keys"], gn, gs, g["num_cells"]).cpu().numpy()
        osel = oracle.poisson_disk_sampling(o["sorted_keys"], on, os_, o["num_cells"])
        assert np.array_equal(sel, osel)
        sel_grid = ops.poisson_disk_sampling_grid(g["sorted_pts"], g["sorted_keys"], g["grid_ds"], g["num_cells"],
                                                  g["cell"]).cpu().numpy()
        assert np.array_equal(sel_grid, osel)


def _neighborhood(pts, ids, num_clouds, radius):
    """Neighbor list of every point in its own cloud, rows mapped to original indices
    (pccnn_lib/pc/Neighborhood.py:27-53 of the reference), from the oracle."""
    cell = np.full((3,), radius, np.float32)
    o = oracle.build_grid(pts, ids, num_clouds, cell)
    keys = oracle.compute_keys(pts, ids, o["aabb_min"], o["num_cells"], cell)
    nb, ends = oracle.find_neighbors(o["sorted_pts"], o["sorted_keys"], pts, keys, o["grid_ds"], o["num_cells"], cell, 0)
    nb = nb.copy()
    nb[:, 0] = o["sorted_ids"][nb[:, 0]].astype(np.int32)
    return nb, ends


def test_single_layer_kpconv_configuration_exactly():
    # 1 cloud of 4096 points uniform in the unit cube, Cin 16, Cout 32, the 16-point table as the layer prepares it,
    # radius 0.1, weights N(0, 1/(15*16)): the CPU-runnable configuration of the benchmark
    from pccnn_lib_b200 import ops
    from pccnn_lib_b200.pc.layers import prepare_kernel_points
    pts = np.random.RandomState(1000).rand(4096, 3).astype(np.float32)
    ids = np.zeros((4096,), np.int32)
    rs = np.random.RandomState(77)
    feats = rs.normal(size=(4096, 16)).astype(np.float32)
    kpts, sigma = prepare_kernel_points(3, 16)
    weights = rs.normal(0, np.sqrt(1.0 / (15 * 16)), size=(16 * 16, 32)).astype(np.float32)
    nb, ends = _neighborhood(pts, ids, 1, 0.1)
    radii = np.full((3,), 0.1, np.float32)
    got = ops.kp_conv(dev(pts), dev(feats), dev(pts), dev(nb), dev(ends), dev(radii), dev(kpts), sigma, dev(weights))
    expect = conv_oracle.kp_conv(pts, feats, pts, nb, ends, radii, kpts, sigma, weights).numpy()
    assert np.isclose(expect, got.cpu().numpy(), rtol=1e-4, atol=1e-4).all()
    # and through the classes, from raw points: Pointcloud -> Grid -> Neighborhood -> KPConv layer
    import pccnn_lib_b200 as lib
    pc = lib.pc.Pointcloud(pts, ids, device=torch.device("cuda:0"))
    layer = lib.pc.layers.KPConv(3, 16, 32, 16).to("cuda:0")
    with torch.no_grad():
        layer.conv_weights_.copy_(dev(weights))
        out, _ = layer(pc, pc, dev(feats), radii)
    assert np.isclose(expect, out.cpu().numpy(), rtol=1e-4, atol=1e-4).all()


def _grads_close(got, expect, tol=2e-4):
    got, expect = np.asarray(got, np.float64), np.asarray(expect, np.float64)
    return float(np.abs(got - expect).max()) <= tol * (np.abs(expect).max() + 1e-30)


@pytest.fixture(scope="module")
def many_samples():
    """140 000 points (two internal chunks of samples, the second one ragged) with about nine neighbors each."""
    n = 140000
    rs = np.random.RandomState(21)
    pts = rs.rand(n, 3).astype(np.float32)
    ids = np.zeros((n,), np.int32)
    nb, ends = _neighborhood(pts, ids, 1, 0.025)
    return dict(pts=pts, nb=nb, ends=ends, radii=np.full((3,), 0.025, np.float32), rs=rs)


def test_kpconv_over_several_sample_chunks(many_samples):
    from pccnn_lib_b200 import ops
    from pccnn_lib_b200.pc.layers import prepare_kernel_points
    c = many_samples
    n, cin, cout, k = c["pts"].shape[0], 8, 24, 8
    rs = np.random.RandomState(5)
    feats = rs.normal(size=(n, cin)).astype(np.float32)
    kpts, sigma = prepare_kernel_points(3, k)
    weights = rs.normal(0, np.sqrt(2.0 / (cin * k)), size=(k * cin, cout)).astype(np.float32)
    a = [dev(c["pts"]), dev(feats), dev(c["pts"]), dev(c["nb"]), dev(c["ends"]), dev(c["radii"])]
    got = ops.kp_conv(*a, dev(kpts), sigma, dev(weights)).cpu().numpy()
    expect = conv_oracle.kp_conv(c["pts"], feats, c["pts"], c["nb"], c["ends"], c["radii"], kpts, sigma, weights).numpy()
    assert np.isclose(expect, got, rtol=1e-4, atol=1e-4).all()
    # the last rows belong to the second, ragged chunk: make sure they were computed at all
    assert np.abs(got[131072:]).max() > 0
    # bf16 inference path over the same chunks
    fb, wb = dev(feats).to(torch.bfloat16), dev(weights).to(torch.bfloat16)
    got16 = ops.kp_conv(a[0], fb, a[2], a[3], a[4], a[5], dev(kpts), sigma, wb).float().cpu().numpy()
    expect16 = conv_oracle.kp_conv(c["pts"], fb.float().cpu().numpy(), c["pts"], c["nb"], c["ends"], c["radii"], kpts,
                                   sigma, wb.float().cpu().numpy()).numpy()
    assert np.abs(got16 - expect16).max() <= 1e-2 * np.abs(expect16).max()
    # gradients (shell points pulled in: see conv_helpers.kp_case)
    kpts_g = (kpts * np.random.RandomState(1).uniform(0.85, 0.99, size=(k, 1))).astype(np.float32)
    g = rs.normal(size=(n, cout)).astype(np.float32)
    got_g = ops.kp_conv_grads(*a, dev(kpts_g), sigma, dev(weights), dev(g))
    expect_g = conv_oracle.kp_conv_grads(c["pts"], feats, c["pts"], c["nb"], c["ends"], c["radii"], kpts_g, sigma,
                                         weights, g)
    for name, x, y in zip(["weights", "features", "kernel_pts", "pts", "samples"], got_g, expect_g):
        assert _grads_close(x.cpu().numpy(), y.numpy()), name


def test_mcconv_over_several_sample_chunks(many_samples):
    from pccnn_lib_b200 import ops
    c = many_samples
    n, cin, cout, h = c["pts"].shape[0], 8, 24, 8
    rs = np.random.RandomState(6)
    feats = rs.normal(size=(n, cin)).astype(np.float32)
    pdf = rs.uniform(0.5, 2.0, size=(n,)).astype(np.float32)
    axis = rs.normal(0, np.sqrt(1 / 3.0), size=(3, h)).astype(np.float32)
    bias = rs.normal(0, 0.1, size=(1, h)).astype(np.float32)
    weights = rs.normal(0, np.sqrt(1.0 / (cin * h)), size=(1, h * cin, cout)).astype(np.float32)
    a = [dev(c["pts"]), dev(pdf), dev(feats), dev(c["pts"]), dev(c["nb"]), dev(c["ends"]), dev(c["radii"]), dev(axis),
         dev(bias), dev(weights)]
    got = ops.mc_conv(*a).cpu().numpy()
    expect = conv_oracle.mc_conv(c["pts"], pdf, feats, c["pts"], c["nb"], c["ends"], c["radii"], axis, bias, weights).numpy()
    scale = max(1.0, float(np.abs(expect).max()))
    assert np.isclose(expect / scale, got / scale, rtol=1e-4, atol=1e-4).all()
    g = rs.normal(size=(n, cout)).astype(np.float32)
    got_g = ops.mc_conv_grads(*a, dev(g))
    expect_g = conv_oracle.mc_conv_grads(c["pts"], pdf, feats, c["pts"], c["nb"], c["ends"], c["radii"], axis, bias,
                                         weights, g)
    for name, x, y in zip(["weights", "features", "axis", "bias", "pdf", "pts", "samples"], got_g, expect_g):
        assert _grads_close(x.cpu().numpy(), y.numpy().reshape(x.shape)), name


@pytest.mark.parametrize("cin", [8, 32])
def test_calls_with_more_than_half_a_million_samples_equal_their_halves(cin):
    """Above 524 288 samples the library switches to chunks of that size (131 072 otherwise).  The rows of a sample do
    not depend on the other samples of the call, so one call over 540 000 samples (one large chunk and a ragged one)
    must give what two calls over its halves give (three small chunks each), which the tests above tie to the oracle:
    bit for bit in the forward pass, within the gradient tolerance where the halves' sums are added.  cin = 8 runs on
    the CUDA cores, cin = 32 through the tensor-core pair kernels."""
    from pccnn_lib_b200 import ops
    from pccnn_lib_b200.pc.layers import prepare_kernel_points
    n, half, cout, k = 540000, 270000, 16, 16
    gen = torch.Generator(device="cuda").manual_seed(3)
    pts = torch.rand((n, 3), device="cuda", generator=gen)
    cell = torch.full((3,), 0.0164, device="cuda")
    g = ops.grid_front_end(pts, torch.zeros((n,), dtype=torch.int32, device="cuda"), 1, cell)
    sp, sk = g["sorted_pts"], g["sorted_keys"]
    nb, ends = ops.find_neighbors(sp, sk, sp, sk, g["grid_ds"], g["num_cells"], cell, 0)
    assert 5 * n < nb.shape[0] < 20 * n
    feats = torch.randn((n, cin), device="cuda", generator=gen)
    kpts, sigma = prepare_kernel_points(3, k)
    kpts = dev((kpts * np.random.RandomState(1).uniform(0.85, 0.99, size=(k, 1))).astype(np.float32))
    weights = torch.randn((k * cin, cout), device="cuda", generator=gen) * float(np.sqrt(2.0 / (cin * k)))
    grads = torch.randn((n, cout), device="cuda", generator=gen)
    t_half = int(ends[half - 1].item())
    parts = [(sp[:half], nb[:t_half], ends[:half], grads[:half]),
             (sp[half:], nb[t_half:] - torch.tensor([0, half], dtype=torch.int32, device="cuda"), ends[half:] - t_half,
              grads[half:])]
    whole = ops.kp_conv(sp, feats, sp, nb, ends, cell, kpts, sigma, weights)
    halves = [ops.kp_conv(sp, feats, s, b.contiguous(), e.contiguous(), cell, kpts, sigma, weights) for s, b, e, _ in parts]
    assert torch.equal(whole, torch.cat(halves, 0))
    assert float(whole[524288:].abs().max()) > 0
    gw = ops.kp_conv_grads(sp, feats, sp, nb, ends, cell, kpts, sigma, weights, grads)
    gh = [ops.kp_conv_grads(sp, feats, s, b.contiguous(), e.contiguous(), cell, kpts, sigma, weights, go.contiguous())
          for s, b, e, go in parts]
    ops.check_status()
    for i, name in enumerate(["weights", "features", "kernel_pts", "pts"]):
        assert _grads_close(gw[i].cpu().numpy(), (gh[0][i] + gh[1][i]).cpu().numpy()), name
    assert _grads_close(gw[4].cpu().numpy(), torch.cat([gh[0][4], gh[1][4]], 0).cpu().numpy()), "samples"


def test_scene_sampler_neighbors_and_capped_density():
    # a small instance of the room-like scene (planes + clutter, density varying over the floor) at its radius
    from pccnn_lib_b200 import ops
    pts = scene_cloud(0, 60000)
    ids = np.zeros((pts.shape[0],), np.int32)
    cell = np.full((3,), 0.25, np.float32)  # 60k points instead of 2M: a wider radius keeps the lists non-trivial
    g = gpu_grid(pts, ids, 1, cell)
    o = oracle.build_grid(pts, ids, 1, cell)
    assert_grid_equal(g, o)
    gn, gs = ops.find_neighbors(g["sorted_pts"], g["sorted_keys"], g["sorted_pts"], g["sorted_keys"], g["grid_ds"],
                                g["num_cells"], g["cell"], 0)
    on, os_ = oracle.find_neighbors(o["sorted_pts"], o["sorted_keys"], o["sorted_pts"], o["sorted_keys"], o["grid_ds"],
                                    o["num_cells"], cell, 0)
    assert np.array_equal(gs.cpu().numpy(), os_) and np.array_equal(gn.cpu().numpy(), on)


def test_shards_reproduce_the_full_batch():
    """A batch split into contiguous cloud ranges (parallel.shard_clouds), every shard processed alone with its batch
    ids renumbered from zero, against the oracle on the WHOLE batch.  The cells per axis are a maximum over the
    clouds of a call, so key values and cell tables differ between a shard and the full batch; cell coordinates,
    neighbor sets, selections and all float results must not."""
    from pccnn_lib_b200 import ops, parallel
    from pccnn_lib_b200.pc.layers import prepare_kernel_points
    spec = [(2, 5000), (13, 9000), (7, 3000), (4, 7000), (9, 4000)]
    pts, ids = _surface_batch(spec)
    sizes = [n for _, n in spec]
    radius = 0.05
    cell = np.full((3,), radius, np.float32)
    first_pt = np.concatenate([[0], np.cumsum(sizes)])
    # full batch, oracle
    o = oracle.build_grid(pts, ids, len(spec), cell)
    on, oe = oracle.find_neighbors(o["sorted_pts"], o["sorted_keys"], o["sorted_pts"], o["sorted_keys"], o["grid_ds"],
                                   o["num_cells"], cell, 0)
    opdf_sorted = oracle.compute_pdf(3, np.full((3,), 0.01, np.float32), o["sorted_pts"], on, oe)
    osel = o["sorted_ids"][oracle.poisson_disk_sampling(o["sorted_keys"], on, oe, o["num_cells"]).reshape(-1)]
    full_pdf = np.empty_like(opdf_sorted)
    full_pdf[o["sorted_ids"]] = opdf_sorted
    onb, oends = _neighborhood(pts, ids, len(spec), radius)  # rows in original indices, samples in original order
    rs = np.random.RandomState(3)
    cin, cout, k = 8, 16, 16
    feats = rs.normal(size=(pts.shape[0], cin)).astype(np.float32)
    kpts, sigma = prepare_kernel_points(3, k)
    weights = rs.normal(0, np.sqrt(2.0 / (cin * k)), size=(k * cin, cout)).astype(np.float32)
    full_out = conv_oracle.kp_conv(pts, feats, pts, onb, oends, cell, kpts, sigma, weights).numpy()

    for world in (2, 3):
        sel_all, seen = [], 0
        for rank in range(world):
            lo, hi = parallel.shard_clouds(sizes, world, rank)
            a, b = int(first_pt[lo]), int(first_pt[hi])
            spts, sids_local = pts[a:b], parallel.rebase_batch_ids(ids[a:b], lo)
            g = gpu_grid(spts, sids_local, hi - lo, cell)
            # against the oracle on the same shard: bit-exact keys and table
            assert_grid_equal(g, oracle.build_grid(spts, sids_local, hi - lo, cell))
            order = g["sorted_ids"].cpu().numpy()
            gn, ge = ops.find_neighbors(g["sorted_pts"], g["sorted_keys"], g["sorted_pts"], g["sorted_keys"],
                                        g["grid_ds"], g["num_cells"], g["cell"], 0)
            pdf_sorted = ops.compute_pdf(3, dev(np.full((3,), 0.01, np.float32)), g["sorted_pts"], gn, ge).cpu().numpy()
            pdf = np.empty_like(pdf_sorted)
            pdf[order] = pdf_sorted
            assert np.allclose(pdf, full_pdf[a:b], rtol=1e-5, atol=0)
            sel = ops.poisson_disk_sampling(g["sorted_keys"], gn, ge, g["num_cells"]).cpu().numpy().reshape(-1)
            sel_all.append(np.sort(order[sel] + a))
            # neighbor sets per point, in original indices of the full batch
            gn_h, ge_h = gn.cpu().numpy(), ge.cpu().numpy()
            starts = np.concatenate([[0], ge_h[:-1]])
            for s_pos in rs.randint(0, b - a, size=200):
                mine = np.sort(order[gn_h[starts[s_pos]:ge_h[s_pos], 0]] + a)
                orig = order[s_pos] + a
                full = np.sort(onb[(oends[orig - 1] if orig > 0 else 0):oends[orig], 0])
                assert np.array_equal(mine, full)
            # convolution of the shard through the classes' route: samples in original order, rows mapped back
            skeys = ops.compute_keys(g["pts"], g["batch_ids"], g["aabb_min"], g["num_cells"], g["cell"])
            cn, ce = ops.find_neighbors(g["sorted_pts"], g["sorted_keys"], g["pts"], skeys, g["grid_ds"], g["num_cells"],
                                        g["cell"], 0, pt_index_map=g["sorted_ids"])
            out = ops.kp_conv(g["pts"], dev(feats[a:b]), g["pts"], cn, ce, g["cell"], dev(kpts), sigma, dev(weights))
            assert np.isclose(full_out[a:b], out.cpu().numpy(), rtol=1e-4, atol=1e-4).all()
            seen += b - a
        assert seen == pts.shape[0]
        assert np.array_equal(np.sort(np.concatenate(sel_all)), np.sort(osel))
