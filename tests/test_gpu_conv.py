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
