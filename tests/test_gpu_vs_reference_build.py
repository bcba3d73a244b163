"""Cross-check against the reference's OWN kernels: the unmodified pccnn_lib_ops sources compiled for
sm_100 by oracle/build_reference.py into oracle/_ref/pccnn_lib_ops.so (built where the reference
sources are available; the built library travels with the repository snapshot, the sources do not).
Skipped when that library is absent."""
import importlib.util
import os

import numpy as np
import pytest
import torch

from conftest import ROOT, ref_case
from conv_helpers import KP_CASES, MC_CASES, kp_case, mc_case
from gpu_helpers import dev, gpu_grid

REF_SO = os.path.join(ROOT, "oracle", "_ref", "pccnn_lib_ops.so")
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.exists(REF_SO), reason="reference build not present")]


@pytest.fixture(scope="module")
def ref_ops():
    spec = importlib.util.spec_from_file_location("pccnn_lib_ops", REF_SO)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def _segments(neigh, ends):
    neigh, ends = neigh.cpu().numpy(), ends.cpu().numpy()
    out, lo = [], 0
    for hi in ends:
        out.append(np.sort(neigh[lo:hi, 0]))
        lo = hi
    return out


@pytest.mark.parametrize("batch_size,num_pts,num_dims,radius", [(16, 1000, 3, 0.2), (16, 1000, 2, 0.2), (4, 1000, 6, 0.2),
                                                               (32, 1000, 3, 0.05)])
def test_keys_table_neighbors_pdf_and_sampling_match_the_reference_kernels(ref_ops, ref_clouds, batch_size, num_pts,
                                                                           num_dims, radius):
    from pccnn_lib_b200 import ops
    pts, batch_ids = ref_case(ref_clouds, batch_size, num_pts, num_dims)
    g = gpu_grid(pts, batch_ids, batch_size, np.full((num_dims,), radius, np.float32))
    # keys and table: bit-exact
    ref_keys = ref_ops.compute_keys(g["pts"], g["batch_ids"], g["aabb_min"], g["num_cells"], g["cell"])
    assert torch.equal(ref_keys, g["keys"])
    shape = [batch_size] + g["num_cells"][0:2].tolist() + [2]
    assert torch.equal(ref_ops.build_grid_ds(g["sorted_keys"], g["num_cells"], shape), g["grid_ds"])
    # neighbor lists: same counts, same sets (the reference's order inside a sample is that of its atomics)
    args = (g["sorted_pts"], g["sorted_keys"], g["sorted_pts"], g["sorted_keys"], g["grid_ds"], g["num_cells"], g["cell"])
    ref_n, ref_s = ref_ops.find_neighbors(*args, 0)
    my_n, my_s = ops.find_neighbors(*args, 0)
    assert torch.equal(ref_s, my_s)
    for a, b in zip(_segments(ref_n, ref_s), _segments(my_n, my_s)):
        assert np.array_equal(a, b)
    # capped search: same counts, and the reference's random subset lies inside our full list
    ref_n4, ref_s4 = ref_ops.find_neighbors(*args, 4)
    my_n4, my_s4 = ops.find_neighbors(*args, 4)
    assert torch.equal(ref_s4, my_s4)
    full = _segments(my_n, my_s)
    for seg_ref, seg_mine, seg_full in zip(_segments(ref_n4, ref_s4), _segments(my_n4, my_s4), full):
        assert np.all(np.isin(seg_ref, seg_full)) and np.all(np.isin(seg_mine, seg_full))
    # KDE on the same list
    bw = dev(np.full((num_dims,), radius * 0.25, np.float32))
    ref_pdf = ref_ops.compute_pdf(num_dims, bw, g["sorted_pts"], my_n, my_s)
    my_pdf = ops.compute_pdf(num_dims, bw, g["sorted_pts"], my_n, my_s)
    assert torch.allclose(ref_pdf, my_pdf, rtol=1e-5, atol=0)
    w = torch.randn(pts.shape[0], device="cuda")
    ref_pg = ref_ops.compute_pdf_grads(num_dims, bw, g["sorted_pts"], my_n, my_s, w)
    my_pg = ops.compute_pdf_grads(num_dims, bw, g["sorted_pts"], my_n, my_s, w)
    assert (ref_pg - my_pg).abs().max() <= 2e-5 * ref_pg.abs().max()
    # Poisson-disk selection: identical
    ref_sel = ref_ops.poisson_disk_sampling(g["sorted_keys"], my_n, my_s, g["num_cells"])
    my_sel = ops.poisson_disk_sampling(g["sorted_keys"], my_n, my_s, g["num_cells"])
    assert torch.equal(ref_sel.reshape(-1), my_sel.reshape(-1))


@pytest.mark.parametrize("c", KP_CASES, ids=lambda c: "d%d_n%d_k%d" % (c["dims"], c["n"], c["k"]))
def test_kpconv_matches_the_reference_kernels(ref_ops, ref_clouds, c):
    from pccnn_lib_b200 import ops
    # forward on the kernel-point table as the layers use it; gradients with the shell points pulled in
    # (self pairs sit exactly on the kink of the clamp otherwise, see conv_helpers.kp_case)
    case = kp_case(ref_clouds, c, normal_feats=True)
    a = [dev(case[k]) for k in ("pts", "feats", "samples", "neighbors", "start_ids", "radii", "kernel_pts")]
    w = dev(case["weights"])
    assert torch.allclose(ref_ops.kp_conv(*a, case["sigma"], w), ops.kp_conv(*a, case["sigma"], w), rtol=1e-4, atol=1e-4)
    case = kp_case(ref_clouds, c, normal_feats=True, shrink=True)
    a = [dev(case[k]) for k in ("pts", "feats", "samples", "neighbors", "start_ids", "radii", "kernel_pts")]
    ref_out = ref_ops.kp_conv(*a, case["sigma"], w)
    g = torch.randn_like(ref_out)
    for name, r, m in zip(["weights", "features", "kernel_pts", "pts", "samples"],
                          ref_ops.kp_conv_grads(*a, case["sigma"], w, g), ops.kp_conv_grads(*a, case["sigma"], w, g)):
        assert (r - m).abs().max() <= 3e-4 * r.abs().max() + 1e-6, name


@pytest.mark.parametrize("c", MC_CASES, ids=lambda c: "d%d_n%d" % (c["dims"], c["n"]))
def test_mcconv_matches_the_reference_kernels(ref_ops, ref_clouds, c):
    from pccnn_lib_b200 import ops
    case = mc_case(ref_clouds, c, normal_feats=True)
    a = [dev(case[k]) for k in ("pts", "pdf", "feats", "samples", "neighbors", "start_ids", "radii", "axis", "bias",
                                "weights")]
    ref_out = ref_ops.mc_conv(*a)
    my_out = ops.mc_conv(*a)
    scale = max(1.0, float(ref_out.abs().max()))
    assert torch.allclose(ref_out / scale, my_out / scale, rtol=1e-4, atol=1e-4)
    g = torch.randn_like(ref_out)
    for name, r, m in zip(["weights", "features", "axis", "bias", "pdf", "pts", "samples"],
                          ref_ops.mc_conv_grads(*a, g), ops.mc_conv_grads(*a, g)):
        assert (r - m.reshape(r.shape)).abs().max() <= 3e-4 * r.abs().max() + 1e-6, name
