"""GPU parity of the weight-variance operators and of KPConvN / PCCNN / SPHConv / PointConv through the C ABI:
against the float64 convolution oracle, and against the reference's own kernels where the compiled reference is
present (the reference has no unit test for any of these operators, so its kernels are the only pin it offers)."""
import importlib.util
import os

import numpy as np
import pytest
import torch

from conftest import ROOT
from conv_helpers import KP_CASES, MC_CASES, kp_case, mc_case
from oracle import conv_oracle

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.as_tensor(np.ascontiguousarray(a), device="cuda")


def close(got, expect, rtol=1e-4, atol=1e-4):
    got, expect = np.asarray(got, np.float64), np.asarray(expect, np.float64)
    scale = max(1.0, float(np.abs(expect).max()))
    return bool(np.isclose(expect / scale, got / scale, rtol=rtol, atol=atol).all())


def grads_close(got, expect, tol=2e-4):
    got, expect = np.asarray(got, np.float64), np.asarray(expect, np.float64)
    return float(np.abs(got - expect).max()) <= tol * (np.abs(expect).max() + 1e-30)


@pytest.fixture(scope="module")
def ref_ops():
    so = os.path.join(ROOT, "oracle", "_ref", "pccnn_lib_ops.so")
    if not os.path.exists(so):
        return None
    spec = importlib.util.spec_from_file_location("pccnn_lib_ops", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _id(c):
    return "d%d_n%d_cin%d_cout%d_k%d" % (c["dims"], c["n"], c["cin"], c["cout"], c["k"])


def _density(case, seed=0):
    return np.random.RandomState(seed).uniform(0.5, 2.0, size=(case["pts"].shape[0],)).astype(np.float32)


# ---- weight variance ------------------------------------------------------------------------------
@pytest.mark.parametrize("c", KP_CASES, ids=_id)
def test_kpconv_weight_variance(ref_clouds, ref_ops, c):
    from pccnn_lib_b200 import ops
    case = kp_case(ref_clouds, c, normal_feats=True)
    keys = ("pts", "feats", "samples", "neighbors", "start_ids", "radii", "kernel_pts")
    got = ops.kp_conv_weight_var(*[dev(case[k]) for k in keys], case["sigma"])
    expect = conv_oracle.kp_conv_weight_var(*[case[k] for k in keys], case["sigma"])
    assert got.dim() == 0 and abs(float(got) - float(expect)) <= 1e-4 * abs(float(expect))
    if ref_ops is not None and c["k"] in (8, 16, 32, 64):
        ref = ref_ops.kp_conv_weight_var(*[dev(case[k]) for k in keys], case["sigma"])
        assert abs(float(got) - float(ref)) <= 1e-4 * abs(float(ref))


@pytest.mark.parametrize("c", MC_CASES, ids=_id)
def test_mcconv_weight_variance(ref_clouds, ref_ops, c):
    from pccnn_lib_b200 import ops
    case = mc_case(ref_clouds, c, normal_feats=True)
    keys = ("pts", "pdf", "feats", "samples", "neighbors", "start_ids", "radii", "axis", "bias")
    got = ops.mc_conv_weight_var(*[dev(case[k]) for k in keys])
    expect = conv_oracle.mc_conv_weight_var(*[case[k] for k in keys])
    assert abs(float(got) - float(expect)) <= 1e-4 * abs(float(expect))
    if ref_ops is not None and c["cin"] % 8 == 0:
        ref = ref_ops.mc_conv_weight_var(*[dev(case[k]) for k in keys])
        assert abs(float(got) - float(ref)) <= 1e-4 * abs(float(ref))


def test_warmup_initialisation_of_the_layers(ref_clouds):
    # pccnn_lib/pc/layers/KPConv.py:103-116 and MCConv.py:97-110: in warm-up state every forward pass re-draws the
    # weights with the variance the batch asks for, so the output variance comes out near the requested one
    import pccnn_lib_b200 as lib
    from conftest import ref_case
    pts, batch_ids = ref_case(ref_clouds, 8, 500, 3)
    device = torch.device("cuda:0")
    pc = lib.pc.Pointcloud(pts, batch_ids, device=device)
    pc.compute_pdf(np.full((3,), 0.1, np.float32))
    torch.manual_seed(1)
    feats = torch.randn(pts.shape[0], 16, device=device)
    radius = np.full((3,), 0.2, np.float32)
    for layer in (lib.pc.layers.KPConv(3, 16, 64, 16, p_constant_weight_var=True),
                  lib.pc.layers.MCConv(3, 16, 64, 16, p_constant_weight_var=True)):
        layer = layer.to(device)
        layer.set_init_warmup_state(True)
        out, nb = layer(pc, pc, feats, radius)
        assert layer.accum_weight_var_ > 0.0
        assert 0.5 < float(out.detach().var()) < 2.0
        layer.set_init_warmup_state(False)
        w = layer.conv_weights_.detach().clone()
        layer(pc, pc, feats, radius, nb)
        assert torch.equal(w, layer.conv_weights_.detach())  # outside warm-up the weights are left alone


# ---- KPConvN / PCCNN ------------------------------------------------------------------------------
@pytest.mark.parametrize("c", KP_CASES, ids=_id)
def test_kpconvn_forward_grads_variance(ref_clouds, ref_ops, c):
    from pccnn_lib_b200 import ops
    case = kp_case(ref_clouds, c, normal_feats=True, shrink=True)
    pdf = _density(case)
    h = [case["pts"], pdf, case["feats"], case["samples"], case["neighbors"], case["start_ids"], case["radii"],
         case["kernel_pts"]]
    a = [dev(x) for x in h]
    w = dev(case["weights"])
    got = ops.kp_conv_n(*a, case["sigma"], w)
    assert close(got.cpu().numpy(), conv_oracle.kp_conv_n(*h, case["sigma"], case["weights"]).numpy())
    g = np.random.RandomState(9).normal(size=(case["samples"].shape[0], c["cout"])).astype(np.float32)
    got_g = ops.kp_conv_n_grads(*a, case["sigma"], w, dev(g))
    for name, x, y in zip(["weights", "features", "kernel_pts", "pts", "samples"], got_g,
                          conv_oracle.kp_conv_n_grads(*h, case["sigma"], case["weights"], g)):
        assert grads_close(x.cpu().numpy(), y.numpy()), name
    var = ops.kp_conv_n_weight_var(*a, case["sigma"])
    expect = conv_oracle.kp_conv_n_weight_var(*h, case["sigma"])
    assert abs(float(var) - float(expect)) <= 1e-4 * abs(float(expect))
    if ref_ops is not None:
        assert torch.allclose(ref_ops.kp_conv_n(*a, case["sigma"], w), got, rtol=1e-4, atol=1e-4 * float(got.abs().max()))
        for name, r, m in zip(["weights", "features", "kernel_pts", "pts", "samples"],
                              ref_ops.kp_conv_n_grads(*a, case["sigma"], w, dev(g)), got_g):
            assert (r - m).abs().max() <= 3e-4 * r.abs().max() + 1e-6, name
        ref_var = ref_ops.kp_conv_n_weight_var(*a, case["sigma"])
        assert abs(float(var) - float(ref_var)) <= 1e-4 * abs(float(ref_var))


@pytest.mark.parametrize("c", KP_CASES, ids=_id)
def test_pccnn_forward_grads_variance(ref_clouds, ref_ops, c):
    from pccnn_lib_b200 import ops
    case = kp_case(ref_clouds, c, normal_feats=True)
    pdf = _density(case, 1)
    sigma = 0.3
    h = [case["pts"], case["feats"], pdf, case["samples"], case["neighbors"], case["start_ids"], case["radii"],
         case["kernel_pts"]]
    a = [dev(x) for x in h]
    w = dev(case["weights"])
    got = ops.pccnn(*a, sigma, w)
    assert close(got.cpu().numpy(), conv_oracle.pccnn(*h, sigma, case["weights"]).numpy())
    g = np.random.RandomState(9).normal(size=(case["samples"].shape[0], c["cout"])).astype(np.float32)
    got_g = ops.pccnn_grads(*a, sigma, w, dev(g))
    for name, x, y in zip(["weights", "features", "kernel_pts", "pdf", "pts", "samples"], got_g,
                          conv_oracle.pccnn_grads(*h, sigma, case["weights"], g)):
        assert grads_close(x.cpu().numpy(), y.numpy()), name
    var = ops.pccnn_weight_variance(*a, sigma)
    expect = conv_oracle.pccnn_weight_variance(*h, sigma)
    assert abs(float(var) - float(expect)) <= 1e-4 * abs(float(expect))
    if ref_ops is not None:
        assert torch.allclose(ref_ops.pccnn(*a, sigma, w), got, rtol=1e-4, atol=1e-4 * float(got.abs().max()))
        for name, r, m in zip(["weights", "features", "kernel_pts", "pdf", "pts", "samples"],
                              ref_ops.pccnn_grads(*a, sigma, w, dev(g)), got_g):
            assert (r - m).abs().max() <= 3e-4 * r.abs().max() + 1e-6, name
        ref_var = ref_ops.pccnn_weight_variance(*a, sigma)
        assert abs(float(var) - float(ref_var)) <= 1e-4 * abs(float(ref_var))


# ---- SPHConv --------------------------------------------------------------------------------------
def _sph_bins(nr, na, npol):
    # equal steps over the ranges the three coordinates really take: (0, 1], (-pi/2, pi/2], (0, pi]
    radial = [(i + 1) / float(nr) for i in range(nr)]
    azimuz = [-np.pi / 2 + (i + 1) * np.pi / float(na) for i in range(na)]
    polar = [(i + 1) * np.pi / float(npol) for i in range(npol)]
    return [np.asarray(x, np.float32) for x in (radial, azimuz, polar)]


@pytest.mark.parametrize("bins", [(1, 5, 3), (2, 4, 3), (3, 7, 3)], ids=lambda b: "%dx%dx%d" % b)
def test_sphconv_forward_grads_variance(ref_clouds, ref_ops, bins):
    from pccnn_lib_b200 import ops
    c = dict(KP_CASES[1], cin=16, cout=24)
    case = kp_case(ref_clouds, c, normal_feats=True)
    radial, azimuz, polar = _sph_bins(*bins)
    k = bins[0] * bins[1] * bins[2] + 1
    weights = np.random.RandomState(4).normal(0, 0.1, size=(k * c["cin"], c["cout"])).astype(np.float32)
    h = [case["pts"], case["feats"], case["samples"], case["neighbors"], case["start_ids"], case["radii"]]
    a = [dev(x) for x in h] + [dev(radial), dev(azimuz), dev(polar)]
    got = ops.sph_conv(*a, dev(weights)).cpu().numpy()
    expect = conv_oracle.sph_conv(*h, radial, azimuz, polar, weights).numpy()
    # a pair whose angle falls within float rounding of a bin edge may be binned differently by the two evaluations:
    # allow a handful of samples to differ, the rest must agree to the usual tolerance
    scale = max(1.0, float(np.abs(expect).max()))
    bad_rows = (~np.isclose(expect / scale, got / scale, rtol=1e-4, atol=1e-4)).any(1)
    assert bad_rows.sum() <= max(2, expect.shape[0] // 500), bad_rows.sum()
    g = np.random.RandomState(9).normal(size=expect.shape).astype(np.float32)
    got_g = ops.sph_conv_grads(*a, dev(weights), dev(g))
    expect_g = conv_oracle.sph_conv_grads(*h, radial, azimuz, polar, weights, g)
    for name, x, y in zip(["weights", "features"], got_g, expect_g):
        assert grads_close(x.cpu().numpy(), y.numpy(), tol=2e-3), name  # tolerance covers an odd re-binned pair
    var = ops.sph_conv_weight_var(*a)
    expect_var = conv_oracle.sph_conv_weight_var(*h, radial, azimuz, polar)
    assert abs(float(var) - float(expect_var)) <= 2e-3 * abs(float(expect_var))
    if ref_ops is not None and k in (8, 16, 32, 64):
        ref = ref_ops.sph_conv(*a, dev(weights)).cpu().numpy()
        bad_rows = (~np.isclose(ref / scale, got / scale, rtol=1e-4, atol=1e-4)).any(1)
        assert bad_rows.sum() <= max(2, ref.shape[0] // 500), bad_rows.sum()
        ref_var = ref_ops.sph_conv_weight_var(*a)
        assert abs(float(var) - float(ref_var)) <= 2e-3 * abs(float(ref_var))


# ---- PointConv ------------------------------------------------------------------------------------
@pytest.mark.parametrize("c", MC_CASES[:4], ids=_id)
def test_pointconv_basis_and_convolution(ref_clouds, ref_ops, c):
    from pccnn_lib_b200 import ops
    case = mc_case(ref_clouds, c, normal_feats=True)
    hb = [case["pts"], case["radii"], case["samples"], case["neighbors"], case["axis"], case["bias"]]
    ab = [dev(x) for x in hb]
    basis = ops.point_conv_basis(*ab)
    expect_basis = conv_oracle.point_conv_basis(*hb).numpy()
    assert np.allclose(basis.cpu().numpy(), expect_basis, rtol=1e-5, atol=1e-5)
    gb = np.random.RandomState(3).normal(size=expect_basis.shape).astype(np.float32)
    for name, x, y in zip(["pts", "samples", "axis", "bias"], ops.point_conv_basis_grads(*ab, dev(gb)),
                          conv_oracle.point_conv_basis_grads(*hb, gb)):
        assert grads_close(x.cpu().numpy(), y.numpy().reshape(x.shape)), name
    # the layer passes the projection through ReLU and a per-pair weight before the convolution; any [T, H] tensor will do
    table = np.maximum(expect_basis, 0.0).astype(np.float32) * np.random.RandomState(5).uniform(
        0.2, 1.0, size=(expect_basis.shape[0], 1)).astype(np.float32)
    weights = case["weights"].reshape(-1, case["weights"].shape[-1])
    hc = [table, case["feats"], case["neighbors"], case["start_ids"]]
    ac = [dev(x) for x in hc]
    got = ops.point_conv(*ac, dev(weights))
    assert close(got.cpu().numpy(), conv_oracle.point_conv(*hc, weights).numpy())
    g = np.random.RandomState(9).normal(size=tuple(got.shape)).astype(np.float32)
    got_g = ops.point_conv_grads(*ac, dev(weights), dev(g))
    for name, x, y in zip(["weights", "features", "basis"], got_g, conv_oracle.point_conv_grads(*hc, weights, g)):
        assert grads_close(x.cpu().numpy(), y.numpy()), name
    var = ops.point_conv_weight_var(*ac)
    expect_var = conv_oracle.point_conv_weight_var(*hc)
    assert abs(float(var) - float(expect_var)) <= 1e-4 * abs(float(expect_var))
    if ref_ops is not None and c["cin"] % 8 == 0:
        assert torch.allclose(ref_ops.point_conv_basis(*ab), basis, rtol=1e-5, atol=1e-5)
        ref = ref_ops.point_conv(*ac, dev(weights))
        assert torch.allclose(ref, got, rtol=1e-4, atol=1e-4 * float(got.abs().max()))
        for name, r, m in zip(["weights", "features", "basis"], ref_ops.point_conv_grads(*ac, dev(weights), dev(g)), got_g):
            assert (r - m).abs().max() <= 3e-4 * r.abs().max() + 1e-6, name
        ref_var = ref_ops.point_conv_weight_var(*ac)
        assert abs(float(var) - float(ref_var)) <= 1e-4 * abs(float(ref_var))


def test_new_layers_run_end_to_end_with_autograd(ref_clouds):
    import pccnn_lib_b200 as lib
    from conftest import ref_case
    pts, batch_ids = ref_case(ref_clouds, 4, 250, 3)
    device = torch.device("cuda:0")
    pc = lib.pc.Pointcloud(pts, batch_ids, device=device)
    pc.compute_pdf(np.full((3,), 0.1, np.float32))
    radius = np.full((3,), 0.2, np.float32)
    torch.manual_seed(0)
    for make in (lambda: lib.pc.layers.KPConvN(3, 8, 16, 16), lambda: lib.pc.layers.PCCNN(3, 8, 16, 16),
                 lambda: lib.pc.layers.SPHConv(3, 8, 16), lambda: lib.pc.layers.PointConv(3, 8, 16, 16),
                 lambda: lib.pc.layers.PointConvFactory(16, True, p_use_bn=True).create_conv_layer(3, 8, 16)):
        layer = make().to(device)
        feats = torch.randn(pts.shape[0], 8, device=device, requires_grad=True)
        layer.set_init_warmup_state(True)
        out, nb = layer(pc, pc, feats, radius)
        layer.set_init_warmup_state(False)
        out = layer(pc, pc, feats, radius, nb)
        out.square().mean().backward()
        assert out.shape == (pts.shape[0], 16) and torch.isfinite(out).all()
        assert feats.grad is not None and torch.isfinite(feats.grad).all() and feats.grad.abs().sum() > 0
        for name, p in layer.named_parameters():
            assert p.grad is not None and torch.isfinite(p.grad).all(), (type(layer).__name__, name)
        assert layer.conv_weights_.grad.abs().sum() > 0
