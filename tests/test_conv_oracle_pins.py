"""Pins the convolution oracle (oracle/conv_oracle.py) to the NumPy expectations of the reference's
own tests and checks its hand-written backward formulas against finite differences."""
import numpy as np
import pytest
import torch

from conv_helpers import KP_CASES, MC_CASES, kp_case, mc_case
from oracle import conv_oracle


def numpy_projection(case, basis, k):
    """unit_test/test_kpconv.py:72-79 of the reference: per-pair outer products into [N, Cin, K]."""
    proj = np.zeros((case["samples"].shape[0], case["feats"].shape[1], k))
    for t in range(case["neighbors"].shape[0]):
        n0, n1 = case["neighbors"][t]
        proj[n1] += case["feats"][n0].reshape(-1, 1) * basis[t].reshape(1, -1)
    return proj.reshape(case["samples"].shape[0], -1)


@pytest.mark.parametrize("c", KP_CASES, ids=lambda c: "d%d_n%d_k%d" % (c["dims"], c["n"], c["k"]))
def test_kpconv_oracle_matches_reference_numpy(ref_clouds, c):
    case = kp_case(ref_clouds, c)
    nb = case["neighbors"]
    # unit_test/test_kpconv.py:60-82
    diff = (case["pts"][nb[:, 0]] - case["samples"][nb[:, 1]]) / case["radii"].reshape(1, -1)
    kd = diff.reshape(-1, 1, c["dims"]) - case["kernel_pts"].reshape(1, -1, c["dims"])
    basis = np.clip(1.0 - np.linalg.norm(kd, axis=-1) / case["sigma"], 0.0, 1.0)
    expect = np.dot(numpy_projection(case, basis, c["k"]), case["weights"])
    got = conv_oracle.kp_conv(case["pts"], case["feats"], case["samples"], nb, case["start_ids"], case["radii"],
                              case["kernel_pts"], case["sigma"], case["weights"]).numpy()
    assert np.isclose(expect, got, rtol=1e-4, atol=1e-4).all()


@pytest.mark.parametrize("c", MC_CASES, ids=lambda c: "d%d_n%d" % (c["dims"], c["n"]))
def test_mcconv_oracle_matches_reference_numpy(ref_clouds, c):
    case = mc_case(ref_clouds, c)
    nb = case["neighbors"]
    # unit_test/test_mcconv.py:65-91
    diff = (case["pts"][nb[:, 0]] - case["samples"][nb[:, 1]]) / case["radii"].reshape(1, -1)
    proj = np.dot(diff, case["axis"]) + case["bias"]
    proj = np.where(proj < 0.0, proj * 0.2, proj) / case["pdf"][nb[:, 0]].reshape(-1, 1)
    expect = np.dot(numpy_projection(case, proj, c["k"]), case["weights"].reshape(c["cin"] * c["k"], -1))
    got = conv_oracle.mc_conv(case["pts"], case["pdf"], case["feats"], case["samples"], nb, case["start_ids"],
                              case["radii"], case["axis"], case["bias"], case["weights"]).numpy()
    assert np.isclose(expect, got, rtol=1e-4, atol=1e-4).all()


def _autograd_check(fn, args, names, in_grads, analytic, tie=None):
    """Gradients of sum(out * in_grads) from torch autograd of the float64 forward against the
    hand-written backward.  Entries where autograd is NaN are skipped: d|x|/dx at x = 0 (a sample
    that is its own neighbor sits exactly on the centre kernel point), where the reference's
    formula returns 0 thanks to its 1e-6 guard."""
    leaves = {n: torch.tensor(np.asarray(args[n], dtype=np.float64), requires_grad=True) for n in names}
    call = dict(args)
    call.update(leaves)
    if tie:  # e.g. samples are the same tensor as pts
        call[tie[0]] = leaves[tie[1]]
    (fn(**call) * torch.as_tensor(in_grads)).sum().backward()
    for n in names:
        auto, ana = leaves[n].grad.numpy(), analytic[n]
        ok = np.isfinite(auto)
        assert ok.mean() > 0.5
        scale = np.abs(auto[ok]).max() + 1e-30
        assert np.abs(auto[ok] - ana[ok]).max() <= 2e-5 * scale, n


def _fd_points_check(fn, args, in_grads, analytic, probes=8, h=1e-6):
    """Central differences with respect to the points when samples are the same array (the
    analytic value is dPts + dSamples).  autograd cannot serve here: every point is its own
    neighbor at distance 0 from the centre kernel point, where sqrt has no derivative."""
    rs = np.random.RandomState(11)
    base = args["pts"].astype(np.float64)
    rest = {k: v for k, v in args.items() if k not in ("pts", "samples")}
    for _ in range(probes):
        idx = (rs.randint(base.shape[0]), rs.randint(base.shape[1]))
        plus, minus = base.copy(), base.copy()
        plus[idx] += h
        minus[idx] -= h
        lp = float((fn(pts=plus, samples=plus, **rest).numpy() * in_grads).sum())
        lm = float((fn(pts=minus, samples=minus, **rest).numpy() * in_grads).sum())
        num = (lp - lm) / (2 * h)
        assert abs(num - analytic[idx]) <= 2e-3 * max(1.0, abs(num)), (idx, num, analytic[idx])  # 1e-6 guard of the reference formula


@pytest.mark.parametrize("c", KP_CASES, ids=lambda c: "d%d_n%d" % (c["dims"], c["n"]))
def test_kpconv_backward_formulas(ref_clouds, c):
    # the reference gradchecks weights, features and kernel points (unit_test/test_kpconv_grads.py:111-121)
    # and points (test_kpconv_pt_grads.py:98-100) numerically in float32; here the hand-written
    # backward is compared with autograd of the float64 forward.
    case = kp_case(ref_clouds, c, normal_feats=True, shrink=True)
    g = np.random.RandomState(3).normal(size=(case["samples"].shape[0], c["cout"]))
    args = dict(pts=case["pts"], feats=case["feats"], samples=case["samples"], neighbors=case["neighbors"],
                start_ids=case["start_ids"], radii=case["radii"], kernel_pts=case["kernel_pts"],
                sigma=case["sigma"], weights=case["weights"])
    dw, df, dk, dp, ds = [t.numpy() for t in conv_oracle.kp_conv_grads(**args, in_grads=g)]
    _autograd_check(conv_oracle.kp_conv, args, ["weights", "feats", "kernel_pts"], g,
                    dict(weights=dw, feats=df, kernel_pts=dk))
    if c["dims"] != 2:  # the 2-D table puts every shell point at distance sigma from the centre: a kink at every self pair
        _fd_points_check(conv_oracle.kp_conv, args, g, dp + ds)


@pytest.mark.parametrize("c", MC_CASES, ids=lambda c: "d%d_n%d" % (c["dims"], c["n"]))
def test_mcconv_backward_formulas(ref_clouds, c):
    # unit_test/test_mcconv_grads.py:127-141 and test_mcconv_pt_grads.py:118-124 of the reference
    case = mc_case(ref_clouds, c, normal_feats=True)
    g = np.random.RandomState(4).normal(size=(case["samples"].shape[0], c["cout"]))
    args = dict(pts=case["pts"], pdf=case["pdf"], feats=case["feats"], samples=case["samples"],
                neighbors=case["neighbors"], start_ids=case["start_ids"], radii=case["radii"], axis=case["axis"],
                bias=case["bias"], weights=case["weights"])
    dw, df, da, db, dpdf, dp, ds = [t.numpy() for t in conv_oracle.mc_conv_grads(**args, in_grads=g)]
    _autograd_check(conv_oracle.mc_conv, args, ["weights", "feats", "axis", "bias", "pdf"], g,
                    dict(weights=dw, feats=df, axis=da, bias=db, pdf=dpdf))
    _autograd_check(conv_oracle.mc_conv, args, ["pts"], g, dict(pts=dp + ds), tie=("samples", "pts"))


def test_mcconv_oracle_with_two_mlps_is_block_diagonal(ref_clouds):
    c = dict(MC_CASES[0], cout=64)
    case = mc_case(ref_clouds, c, num_mlps=2)
    got = conv_oracle.mc_conv(case["pts"], case["pdf"], case["feats"], case["samples"], case["neighbors"],
                              case["start_ids"], case["radii"], case["axis"], case["bias"], case["weights"])
    assert tuple(got.shape) == (case["samples"].shape[0], 64) and torch.isfinite(got).all()


@pytest.mark.parametrize("dims", [2, 3, 4])
@pytest.mark.parametrize("num_pts", [8, 16, 32, 64])
def test_prepared_kernel_points_are_the_reference_layers(dims, num_pts):
    # kernel_pts_ / sigma_ of a fresh KPConv layer against what the reference's constructor registers
    # (pccnn_lib/pc/layers/KPConv.py:45-57), stored by oracle/make_kernel_points.py from the reference install
    import os
    from conftest import GOLDEN
    from pccnn_lib_b200.pc.layers import prepare_kernel_points
    golden = np.load(os.path.join(GOLDEN, "ref_kernel_points_prepared.npz"))
    pts, sigma = prepare_kernel_points(dims, num_pts)
    assert pts.dtype == np.float32 and np.array_equal(pts, golden["%d_%d_pts" % (dims, num_pts)])
    assert sigma == float(golden["%d_%d_sigma" % (dims, num_pts)])


def test_weight_variance_double_sum_is_the_norm_of_the_projected_features(ref_clouds):
    # pcconvs/shared/compute_variance_weights.cu:49-88 loops over all pairs (i, j) of a sample's neighbors; the CUDA
    # implementation evaluates the same quantity as the squared norm of the sample's projected features
    case = kp_case(ref_clouds, KP_CASES[0], normal_feats=True)
    keys = ("pts", "feats", "samples", "neighbors", "start_ids", "radii", "kernel_pts")
    var = conv_oracle.kp_conv_weight_var(*[case[k] for k in keys], case["sigma"])
    t = lambda k: torch.as_tensor(case[k]).double()
    nb = torch.as_tensor(case["neighbors"])
    basis = conv_oracle.kernel_pts_basis(conv_oracle.pt_diff(t("pts"), t("samples"), nb, t("radii")), t("kernel_pts"),
                                         case["sigma"])
    proj = conv_oracle.feat_basis_proj(basis, t("feats"), nb, case["samples"].shape[0])
    assert abs(float(var) - float(1.0 / (proj.reshape(proj.shape[0], -1) ** 2).sum(1).mean())) <= 1e-12 * abs(float(var))


@pytest.mark.parametrize("c", KP_CASES[:2], ids=lambda c: "d%d_n%d" % (c["dims"], c["n"]))
def test_density_normalised_kernel_point_backward_formulas(ref_clouds, c):
    # pcconvs/pccnn.cu:69-139 and kpconvn.cu:71-130 restated by hand against autograd of the float64 forward
    case = kp_case(ref_clouds, c, normal_feats=True, shrink=True)
    pdf = np.random.RandomState(0).uniform(0.5, 2.0, size=case["pts"].shape[0])
    g = np.random.RandomState(1).normal(size=(case["samples"].shape[0], c["cout"]))
    args = dict(pts=case["pts"], feats=case["feats"], pdf=pdf, samples=case["samples"], neighbors=case["neighbors"],
                start_ids=case["start_ids"], radii=case["radii"], kernel_pts=case["kernel_pts"], sigma=0.3,
                weights=case["weights"])
    dw, df, dk, dpdf, dp, ds = [x.numpy() for x in conv_oracle.pccnn_grads(**args, in_grads=g)]
    _autograd_check(conv_oracle.pccnn, args, ["weights", "feats", "kernel_pts", "pdf"], g,
                    dict(weights=dw, feats=df, kernel_pts=dk, pdf=dpdf))
    _autograd_check(conv_oracle.pccnn, args, ["pts"], g, dict(pts=dp + ds), tie=("samples", "pts"))
    args["sigma"] = case["sigma"]
    dw, df, dk, dp, ds = [x.numpy() for x in conv_oracle.kp_conv_n_grads(**args, in_grads=g)]
    _autograd_check(conv_oracle.kp_conv_n, args, ["weights", "feats", "kernel_pts"], g,
                    dict(weights=dw, feats=df, kernel_pts=dk))


def test_spherical_basis_is_one_hot_and_sphconv_averages(ref_clouds):
    case = kp_case(ref_clouds, KP_CASES[1])
    t = lambda k: torch.as_tensor(case[k]).double()
    nb = torch.as_tensor(case["neighbors"])
    diffs = conv_oracle.pt_diff(t("pts"), t("samples"), nb, t("radii"))
    basis = conv_oracle.spherical_basis(diffs, [0.5, 1.0], [-0.5, 0.5, 1.6], [1.0, 2.0, 3.2])
    assert tuple(basis.shape) == (nb.shape[0], 19) and bool((basis.sum(1) == 1.0).all())
    self_pairs = (nb[:, 0] == nb[:, 1])
    assert bool((basis[self_pairs, 0] == 1.0).all()) and float(basis[~self_pairs, 0].sum()) == 0.0
    # with all-ones features and weights every output is (neighbors * Cin) / (neighbors + 1e-6)
    ones_f = np.ones((case["pts"].shape[0], 2), np.float32)
    w = np.ones((19 * 2, 3), np.float32)
    out = conv_oracle.sph_conv(case["pts"], ones_f, case["samples"], case["neighbors"], case["start_ids"], case["radii"],
                               [0.5, 1.0], [-0.5, 0.5, 1.6], [1.0, 2.0, 3.2], w)
    assert np.allclose(out.numpy(), 2.0, rtol=1e-5)
