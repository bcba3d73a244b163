"""GPU parity of KPConv / MCConv (forward and gradients) through the C ABI against the float64
convolution oracle, on the reference's own test cases and on shapes it cannot run."""
import numpy as np
import pytest
import torch

from conv_helpers import EXTRA_KP_CASES, KP_CASES, MC_CASES, kp_case, mc_case
from oracle import conv_oracle

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.as_tensor(np.ascontiguousarray(a), device="cuda")


def close(got, expect, rtol=1e-4, atol=1e-4):
    """The reference's own criterion (unit_test/test_kpconv.py:84): isclose(rtol=1e-4, atol=1e-4)."""
    got, expect = np.asarray(got, np.float64), np.asarray(expect, np.float64)
    return bool(np.isclose(expect, got, rtol=rtol, atol=atol).all())


def _id(c):
    return "d%d_n%d_cin%d_cout%d_k%d" % (c["dims"], c["n"], c["cin"], c["cout"], c["k"])


@pytest.mark.parametrize("c", KP_CASES + EXTRA_KP_CASES, ids=_id)
def test_kpconv_forward(ref_clouds, c):
    from pccnn_lib_b200 import ops
    case = kp_case(ref_clouds, c)
    got = ops.kp_conv(dev(case["pts"]), dev(case["feats"]), dev(case["samples"]), dev(case["neighbors"]),
                      dev(case["start_ids"]), dev(case["radii"]), dev(case["kernel_pts"]), case["sigma"],
                      dev(case["weights"])).cpu().numpy()
    expect = conv_oracle.kp_conv(case["pts"], case["feats"], case["samples"], case["neighbors"], case["start_ids"],
                                 case["radii"], case["kernel_pts"], case["sigma"], case["weights"]).numpy()
    assert close(got, expect)


@pytest.mark.parametrize("c", MC_CASES, ids=_id)
@pytest.mark.parametrize("num_mlps", [1, 2])
def test_mcconv_forward(ref_clouds, c, num_mlps):
    from pccnn_lib_b200 import ops
    if num_mlps == 2:
        c = dict(c, cout=max(c["cout"], 8), cin=32)
    case = mc_case(ref_clouds, c, num_mlps=num_mlps)
    got = ops.mc_conv(dev(case["pts"]), dev(case["pdf"]), dev(case["feats"]), dev(case["samples"]),
                      dev(case["neighbors"]), dev(case["start_ids"]), dev(case["radii"]), dev(case["axis"]),
                      dev(case["bias"]), dev(case["weights"])).cpu().numpy()
    expect = conv_oracle.mc_conv(case["pts"], case["pdf"], case["feats"], case["samples"], case["neighbors"],
                                 case["start_ids"], case["radii"], case["axis"], case["bias"], case["weights"]).numpy()
    # MCConv outputs scale with 1/pdf: compare relative to the output's magnitude as well
    scale = max(1.0, float(np.abs(expect).max()))
    assert close(got / scale, expect / scale)


def grads_close(got, expect, tol=2e-4):
    """Gradients are compared relative to the largest entry of the tensor: sums of thousands of
    float reductions in arbitrary order against a float64 oracle."""
    got, expect = np.asarray(got, np.float64), np.asarray(expect, np.float64)
    scale = np.abs(expect).max() + 1e-30
    return float(np.abs(got - expect).max()) <= tol * scale


@pytest.mark.parametrize("c", KP_CASES + EXTRA_KP_CASES[:3], ids=_id)
def test_kpconv_grads(ref_clouds, c):
    from pccnn_lib_b200 import ops
    case = kp_case(ref_clouds, c, normal_feats=True, shrink=True)
    g = np.random.RandomState(9).normal(size=(case["samples"].shape[0], c["cout"])).astype(np.float32)
    got = ops.kp_conv_grads(dev(case["pts"]), dev(case["feats"]), dev(case["samples"]), dev(case["neighbors"]),
                            dev(case["start_ids"]), dev(case["radii"]), dev(case["kernel_pts"]), case["sigma"],
                            dev(case["weights"]), dev(g))
    expect = conv_oracle.kp_conv_grads(case["pts"], case["feats"], case["samples"], case["neighbors"],
                                       case["start_ids"], case["radii"], case["kernel_pts"], case["sigma"],
                                       case["weights"], g)
    for name, a, b in zip(["weights", "features", "kernel_pts", "pts", "samples"], got, expect):
        assert grads_close(a.cpu().numpy(), b.numpy()), name


@pytest.mark.parametrize("c", MC_CASES, ids=_id)
def test_mcconv_grads(ref_clouds, c):
    from pccnn_lib_b200 import ops
    case = mc_case(ref_clouds, c, normal_feats=True)
    g = np.random.RandomState(10).normal(size=(case["samples"].shape[0], c["cout"])).astype(np.float32)
    got = ops.mc_conv_grads(dev(case["pts"]), dev(case["pdf"]), dev(case["feats"]), dev(case["samples"]),
                            dev(case["neighbors"]), dev(case["start_ids"]), dev(case["radii"]), dev(case["axis"]),
                            dev(case["bias"]), dev(case["weights"]), dev(g))
    expect = conv_oracle.mc_conv_grads(case["pts"], case["pdf"], case["feats"], case["samples"], case["neighbors"],
                                       case["start_ids"], case["radii"], case["axis"], case["bias"], case["weights"], g)
    for name, a, b in zip(["weights", "features", "axis", "bias", "pdf", "pts", "samples"], got, expect):
        assert grads_close(a.cpu().numpy(), b.numpy().reshape(a.shape)), name


@pytest.mark.parametrize("num_mlps,cout", [(2, 64), (4, 64), (2, 16), (4, 96)])
def test_mcconv_with_several_mlps_forward_and_grads(ref_clouds, num_mlps, cout):
    # per-MLP slices of the projected operand, of the weights and of the upstream gradient, including output
    # slices narrower than one 64-column tensor-core tile (e.g. MCConv(cin=32, cout=64, hidden=16, mlps=4))
    from pccnn_lib_b200 import ops
    c = dict(MC_CASES[0], cout=cout)
    case = mc_case(ref_clouds, c, normal_feats=True, num_mlps=num_mlps)
    a = [dev(case[k]) for k in ("pts", "pdf", "feats", "samples", "neighbors", "start_ids", "radii", "axis", "bias",
                                "weights")]
    h = [case[k] for k in ("pts", "pdf", "feats", "samples", "neighbors", "start_ids", "radii", "axis", "bias", "weights")]
    got = ops.mc_conv(*a).cpu().numpy()
    expect = conv_oracle.mc_conv(*h).numpy()
    scale = max(1.0, float(np.abs(expect).max()))
    assert close(got / scale, expect / scale)
    g = np.random.RandomState(11).normal(size=(case["samples"].shape[0], cout)).astype(np.float32)
    for name, x, y in zip(["weights", "features", "axis", "bias", "pdf", "pts", "samples"],
                          ops.mc_conv_grads(*a, dev(g)), conv_oracle.mc_conv_grads(*h, g)):
        assert grads_close(x.cpu().numpy(), y.numpy().reshape(x.shape)), name


def test_layers_run_end_to_end_with_autograd(ref_clouds):
    # The mirrored classes: Pointcloud -> compute_pdf -> MCConv / KPConv -> backward through the op wrappers.
    import pccnn_lib_b200 as lib
    from conftest import ref_case
    pts, batch_ids = ref_case(ref_clouds, 4, 250, 3)
    device = torch.device("cuda:0")
    pc = lib.pc.Pointcloud(pts, batch_ids, device=device)
    feats = torch.randn(pts.shape[0], 8, device=device, requires_grad=True)
    radius = np.full((3,), 0.2, np.float32)
    pc.compute_pdf(np.full((3,), 0.1, np.float32))
    torch.manual_seed(0)
    kp = lib.pc.layers.KPConv(3, 8, 16, 16).to(device)
    mc = lib.pc.layers.MCConv(3, 16, 8, 16).to(device)
    out1, neighborhood = kp(pc, pc, feats, radius)
    out2 = mc(pc, pc, out1, radius, neighborhood)
    out2.square().mean().backward()
    assert out2.shape == (pts.shape[0], 8) and torch.isfinite(out2).all()
    for p in [feats, kp.conv_weights_, mc.conv_weights_, mc.proj_axis_, mc.proj_bias_]:
        assert p.grad is not None and torch.isfinite(p.grad).all() and p.grad.abs().sum() > 0


@pytest.mark.parametrize("c", [KP_CASES[0], EXTRA_KP_CASES[0], EXTRA_KP_CASES[2]], ids=_id)
def test_kpconv_bf16_inference_path(ref_clouds, c):
    # bf16 features / weights / output, fp32 accumulation: within 1e-2 of the float64 oracle evaluated on
    # the bf16-rounded inputs (relative to the output's magnitude).
    from pccnn_lib_b200 import ops
    case = kp_case(ref_clouds, c, normal_feats=True)
    feats = dev(case["feats"]).to(torch.bfloat16)
    weights = dev(case["weights"]).to(torch.bfloat16)
    got = ops.kp_conv(dev(case["pts"]), feats, dev(case["samples"]), dev(case["neighbors"]), dev(case["start_ids"]),
                      dev(case["radii"]), dev(case["kernel_pts"]), case["sigma"], weights)
    assert got.dtype == torch.bfloat16
    expect = conv_oracle.kp_conv(case["pts"], feats.float().cpu().numpy(), case["samples"], case["neighbors"],
                                 case["start_ids"], case["radii"], case["kernel_pts"], case["sigma"],
                                 weights.float().cpu().numpy()).numpy()
    scale = np.abs(expect).max()
    assert np.abs(got.float().cpu().numpy() - expect).max() <= 1e-2 * scale
