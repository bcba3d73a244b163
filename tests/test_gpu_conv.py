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


def close_to_scale(got, expect, tol=1e-4):
    """Within 1e-4 of the output's magnitude: the criterion for neighborhoods of hundreds of points, where sums of
    ~10^6 float32 products leave an absolute error that the per-element criterion above (made for the reference's
    small test clouds) does not allow for outputs near zero -- on either kernel path, and in the reference's own
    float32 kernels alike."""
    got, expect = np.asarray(got, np.float64), np.asarray(expect, np.float64)
    return float(np.abs(got - expect).max()) <= tol * max(1.0, float(np.abs(expect).max()))


def _id(c):
    return "d%d_n%d_cin%d_cout%d_k%d" % (c["dims"], c["n"], c["cin"], c["cout"], c["k"])


# many neighbors per sample (several 128-neighbor passes) and more than 128 channels (several channel blocks)
DENSE_KP_CASES = [dict(seed=12, batch=1, n=1000, dims=3, cin=136, cout=24, k=16, radius=0.5),
                  dict(seed=13, batch=1, n=1000, dims=3, cin=32, cout=24, k=16, radius=0.5)]


@pytest.mark.parametrize("c", KP_CASES + EXTRA_KP_CASES + DENSE_KP_CASES, ids=_id)
def test_kpconv_forward(ref_clouds, c):
    from pccnn_lib_b200 import ops
    case = kp_case(ref_clouds, c)
    got = ops.kp_conv(dev(case["pts"]), dev(case["feats"]), dev(case["samples"]), dev(case["neighbors"]),
                      dev(case["start_ids"]), dev(case["radii"]), dev(case["kernel_pts"]), case["sigma"],
                      dev(case["weights"])).cpu().numpy()
    expect = conv_oracle.kp_conv(case["pts"], case["feats"], case["samples"], case["neighbors"], case["start_ids"],
                                 case["radii"], case["kernel_pts"], case["sigma"], case["weights"]).numpy()
    assert close_to_scale(got, expect) if c in DENSE_KP_CASES else close(got, expect)


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


@pytest.mark.parametrize("c", KP_CASES + EXTRA_KP_CASES[:3] + DENSE_KP_CASES, ids=_id)
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
        # with ~10^6 pairs a few sit within float rounding of the kink of clamp(1 - dist / sigma), where the float32 and
        # the float64 evaluation take different branches of the derivative: the geometric gradients of the dense cases
        # get the room of a few such pairs (both kernel paths and the reference's float32 kernels behave alike)
        tol = 2e-3 if (c in DENSE_KP_CASES and name in ("kernel_pts", "pts", "samples")) else 2e-4
        assert grads_close(a.cpu().numpy(), b.numpy(), tol), name


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


LIST_FREE_CASES = [dict(seed=33, batch=4, n=250, dims=3, cin=32, cout=64, k=16, radius=0.25),
                   dict(seed=5, batch=3, n=400, dims=3, cin=3, cout=64, k=16, radius=0.2),
                   dict(seed=7, batch=2, n=500, dims=3, cin=70, cout=130, k=32, radius=0.15, pooled=True),
                   dict(seed=6, batch=2, n=300, dims=3, cin=20, cout=10, k=15, radius=0.2),
                   # more than 128 neighbors per sample (several passes per sample) and more than 128 channels
                   dict(seed=12, batch=1, n=1000, dims=3, cin=136, cout=24, k=16, radius=0.5),
                   dict(seed=13, batch=1, n=1000, dims=3, cin=32, cout=24, k=16, radius=0.5),
                   dict(seed=14, batch=2, n=400, dims=3, cin=136, cout=24, k=16, radius=0.15)]


@pytest.mark.parametrize("c", LIST_FREE_CASES, ids=_id)
@pytest.mark.parametrize("bf16", [False, True], ids=["f32", "bf16"])
def test_kpconv_without_a_neighbor_list(ref_clouds, c, bf16):
    # the list-free operator against the float64 oracle evaluated on the oracle's own neighbor list
    from gpu_helpers import gpu_grid
    from pccnn_lib_b200 import ops
    case = kp_case(ref_clouds, c, normal_feats=True)
    g = gpu_grid(case["pts"], case["batch_ids"], c["batch"], case["radii"])
    samples = dev(case["samples"])
    sample_b = case["sample_batch_ids"]
    skeys = ops.compute_keys(samples, dev(sample_b), g["aabb_min"], g["num_cells"], g["cell"])
    feats, weights = dev(case["feats"]), dev(case["weights"])
    if bf16:
        feats, weights = feats.to(torch.bfloat16), weights.to(torch.bfloat16)
    got = ops.kp_conv_grid(g["sorted_pts"], g["sorted_keys"], g["sorted_ids"], feats, samples, skeys, g["grid_ds"],
                           g["num_cells"], g["cell"], dev(case["kernel_pts"]), case["sigma"], weights)
    expect = conv_oracle.kp_conv(case["pts"], feats.float().cpu().numpy(), case["samples"], case["neighbors"],
                                 case["start_ids"], case["radii"], case["kernel_pts"], case["sigma"],
                                 weights.float().cpu().numpy()).numpy()
    if bf16:
        assert got.dtype == torch.bfloat16
        assert np.abs(got.float().cpu().numpy() - expect).max() <= 1e-2 * np.abs(expect).max()
    else:
        assert close_to_scale(got.cpu().numpy(), expect)
        # and identical (to rounding) to the list-based operator on the GPU's own list
        nb, ends = ops.find_neighbors(g["sorted_pts"], g["sorted_keys"], samples, skeys, g["grid_ds"], g["num_cells"],
                                      g["cell"], 0, pt_index_map=g["sorted_ids"])
        listed = ops.kp_conv(dev(case["pts"]), feats, samples, nb, ends, g["cell"], dev(case["kernel_pts"]), case["sigma"],
                             weights)
        assert close_to_scale(got.cpu().numpy(), listed.cpu().numpy())


def test_kpconv_layer_accepts_a_grid_neighborhood(ref_clouds):
    import pccnn_lib_b200 as lib
    from conftest import ref_case
    pts, batch_ids = ref_case(ref_clouds, 4, 250, 3)
    device = torch.device("cuda:0")
    pc = lib.pc.Pointcloud(pts, batch_ids, device=device)
    radius = torch.full((3,), 0.2, device=device)
    grid = lib.pc.Grid(pc, lib.pc.BoundingBox(pc), radius)
    grid.compute_cell_ids()
    grid.build_ds()
    torch.manual_seed(0)
    layer = lib.pc.layers.KPConv(3, 8, 16, 16).to(device)
    feats = torch.randn(pts.shape[0], 8, device=device)
    with torch.no_grad():
        listed = layer(pc, pc, feats, radius, lib.pc.Neighborhood(grid, pc, 0))
        free = layer(pc, pc, feats, radius, lib.pc.GridNeighborhood(grid, pc))
    assert torch.allclose(listed, free, rtol=1e-4, atol=1e-4)
    with pytest.raises(RuntimeError, match="neighbor list"):
        layer(pc, pc, feats.requires_grad_(True), radius, lib.pc.GridNeighborhood(grid, pc))
