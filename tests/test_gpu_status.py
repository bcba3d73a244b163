"""Failure reporting and input validation on the GPU (no counterpart in the reference, which checks nothing):
a bounded wait that runs out must end in an error code on the host with the context still usable, and a
malformed neighbor list must be refused instead of read.

The waits are made to run out in the harmless way: a test hook tells the producer thread of the tensor-core kernels
to issue no load from the second K block on, so the consumers wait on a barrier that nothing will ever flip while no
copy is in flight; the poll limit is lowered so that this takes microseconds."""
import numpy as np
import pytest
import torch

from conv_helpers import KP_CASES, kp_case
from oracle import conv_oracle

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.as_tensor(np.ascontiguousarray(a), device="cuda")


class short_waits_and_a_silent_producer(object):
    def __enter__(self):
        from pccnn_lib_b200 import _capi
        _capi.check(_capi.lib.pccnn_gemm_set_test_hooks(4000, 1), "set_test_hooks")

    def __exit__(self, *exc):
        from pccnn_lib_b200 import _capi
        torch.cuda.synchronize()
        _capi.check(_capi.lib.pccnn_gemm_set_test_hooks(0, -1), "set_test_hooks")
        return False


@pytest.mark.parametrize("shape", [(300, 96, 256), (128 * 200, 64, 192)], ids=["tile_per_cta", "persistent"])
def test_contraction_reports_a_wait_that_ran_out_and_recovers(shape):
    from pccnn_lib_b200 import ops
    m, n, k = shape
    rs = np.random.RandomState(0)
    a, b = dev(rs.normal(size=(m, k)).astype(np.float32)), dev(rs.normal(size=(n, k)).astype(np.float32))
    with short_waits_and_a_silent_producer():
        with pytest.raises(RuntimeError, match="bounded wait"):
            ops.gemm_f32(a, b)
    got = ops.gemm_f32(a, b).cpu().numpy().astype(np.float64)  # same context, hooks off: normal result
    expect = a.cpu().numpy().astype(np.float64) @ b.cpu().numpy().astype(np.float64).T
    assert np.abs(got - expect).max() <= 1e-4 * np.abs(expect).max()


def test_weight_gradient_contraction_reports_a_wait_that_ran_out_and_recovers():
    from pccnn_lib_b200 import ops
    rs = np.random.RandomState(1)
    a, b = dev(rs.normal(size=(1000, 200)).astype(np.float32)), dev(rs.normal(size=(1000, 72)).astype(np.float32))
    with short_waits_and_a_silent_producer():
        with pytest.raises(RuntimeError, match="bounded wait"):
            ops.gemm_tn_f32(a, b)
    got = ops.gemm_tn_f32(a, b).cpu().numpy().astype(np.float64)
    expect = a.cpu().numpy().astype(np.float64).T @ b.cpu().numpy().astype(np.float64)
    assert np.abs(got - expect).max() <= 1e-4 * np.abs(expect).max()


def test_convolution_surfaces_the_failure_of_its_contraction(ref_clouds):
    from pccnn_lib_b200 import ops
    case = kp_case(ref_clouds, KP_CASES[0])
    args = [dev(case[k]) for k in ("pts", "feats", "samples", "neighbors", "start_ids", "radii", "kernel_pts")]
    w = dev(case["weights"])
    ops.check_status()  # nothing pending
    with short_waits_and_a_silent_producer():
        ops.kp_conv(*args, case["sigma"], w)  # asynchronous: the call itself cannot know yet
        with pytest.raises(RuntimeError, match="gave up"):
            ops.check_status(synchronize=True)
    ops.check_status()  # the record was consumed
    # a failure that nobody asked about is found by the next convolution call
    with short_waits_and_a_silent_producer():
        ops.kp_conv(*args, case["sigma"], w)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="gave up"):
        ops.kp_conv(*args, case["sigma"], w)
    got = ops.kp_conv(*args, case["sigma"], w).cpu().numpy()
    expect = conv_oracle.kp_conv(case["pts"], case["feats"], case["samples"], case["neighbors"], case["start_ids"],
                                 case["radii"], case["kernel_pts"], case["sigma"], case["weights"]).numpy()
    assert np.isclose(expect, got, rtol=1e-4, atol=1e-4).all()
    ops.check_status()


def test_malformed_neighbor_lists_are_refused(ref_clouds):
    from pccnn_lib_b200 import ops
    case = kp_case(ref_clouds, KP_CASES[0])
    n = case["pts"].shape[0]
    nb, ends = case["neighbors"].copy(), case["start_ids"].copy()
    ops.validate_neighbors(dev(nb), dev(ends), n)  # the real list passes

    bad = nb.copy()
    bad[17, 0] = n  # one past the last point
    with pytest.raises(RuntimeError, match="point index"):
        ops.validate_neighbors(dev(bad), dev(ends), n)
    bad = nb.copy()
    bad[5, 0] = -1
    with pytest.raises(RuntimeError, match="point index"):
        ops.validate_neighbors(dev(bad), dev(ends), n)
    bad = nb.copy()
    bad[40, 1] += 1  # row stored in another sample's segment
    with pytest.raises(RuntimeError, match="sample index"):
        ops.validate_neighbors(dev(bad), dev(ends), n)
    bad_ends = ends.copy()
    bad_ends[10] = bad_ends[9] - 1
    with pytest.raises(RuntimeError, match="decrease"):
        ops.validate_neighbors(dev(nb), dev(bad_ends), n)
    bad_ends = ends.copy()
    bad_ends[-1] += 3
    with pytest.raises(RuntimeError, match="last end offset"):
        ops.validate_neighbors(dev(nb), dev(bad_ends), n)
    # empty list, empty samples
    ops.validate_neighbors(dev(np.zeros((0, 2), np.int32)), dev(np.zeros((4,), np.int32)), n)


def test_operators_validate_their_lists_when_asked(ref_clouds, monkeypatch):
    from pccnn_lib_b200 import ops
    case = kp_case(ref_clouds, KP_CASES[0])
    bad = case["neighbors"].copy()
    bad[3, 0] = 10 ** 6
    monkeypatch.setenv("PCCNN_VALIDATE_NEIGHBORS", "1")
    args = [dev(case["pts"]), dev(case["feats"]), dev(case["samples"]), dev(bad), dev(case["start_ids"]),
            dev(case["radii"]), dev(case["kernel_pts"])]
    with pytest.raises(RuntimeError, match="point index"):
        ops.kp_conv(*args, case["sigma"], dev(case["weights"]))
    with pytest.raises(RuntimeError, match="point index"):
        ops.compute_pdf(3, dev(np.full((3,), 0.1, np.float32)), dev(case["pts"]), dev(bad), dev(case["start_ids"]))
