"""GPU parity of the tcgen05 contraction against a float64 NumPy product."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(128, 128, 64), (300, 64, 256), (1000, 4, 512), (257, 200, 2048), (500, 600, 128), (64, 32, 48),
          (4096, 128, 2048), (1, 16, 64), (129, 17, 100),
          # more output tiles than SMs: the persistent kernel with the double-buffered accumulator
          (40000, 128, 192), (30000, 300, 128), (25000, 40, 320), (20001, 16, 64)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_split_gemm_has_fp32_accuracy(m, n, k):
    from pccnn_lib_b200 import ops
    rs = np.random.RandomState(m + n + k)
    a = rs.randn(m, k).astype(np.float32)
    b = rs.randn(n, k).astype(np.float32)
    got = ops.gemm_f32(torch.as_tensor(a, device="cuda"), torch.as_tensor(b, device="cuda"), split=True).cpu().numpy()
    expect = a.astype(np.float64) @ b.astype(np.float64).T
    # hi/lo split drops products below 2^-16 of each term: error relative to |a|.|b| stays under 1e-5
    bound = (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64).T) * 5e-5 + 1e-6  # worst case 3 * 2^-16 per product (bf16 unit roundoff 2^-8)
    assert np.all(np.abs(got - expect) <= bound)
    assert np.allclose(got, expect, rtol=1e-4, atol=1e-4 * np.sqrt(k))


@pytest.mark.parametrize("m,n,k", SHAPES[:5] + SHAPES[-4:-2])
def test_single_pass_gemm_matches_bf16_rounded_inputs(m, n, k):
    from pccnn_lib_b200 import ops
    rs = np.random.RandomState(7 * m + n + k)
    a = rs.randn(m, k).astype(np.float32)
    b = rs.randn(n, k).astype(np.float32)
    ta, tb = torch.as_tensor(a, device="cuda"), torch.as_tensor(b, device="cuda")
    got = ops.gemm_f32(ta, tb, split=False).cpu().numpy()
    ar = ta.to(torch.bfloat16).to(torch.float64).cpu().numpy()
    br = tb.to(torch.bfloat16).to(torch.float64).cpu().numpy()
    expect = ar @ br.T
    assert np.allclose(got, expect, rtol=1e-5, atol=1e-5 * np.sqrt(k) * 4)


TN_SHAPES = [(64, 128, 64), (1000, 256, 128), (5000, 2048, 128), (300, 48, 4), (4097, 512, 300), (1, 64, 64),
             (70000, 128, 64)]


@pytest.mark.parametrize("rows,i,n", TN_SHAPES)
def test_split_gemm_tn_has_fp32_accuracy(rows, i, n):
    from pccnn_lib_b200 import ops
    rs = np.random.RandomState(rows + i + n)
    a = rs.randn(rows, i).astype(np.float32)
    b = rs.randn(rows, n).astype(np.float32)
    got = ops.gemm_tn_f32(torch.as_tensor(a, device="cuda"), torch.as_tensor(b, device="cuda")).cpu().numpy()
    expect = a.astype(np.float64).T @ b.astype(np.float64)
    bound = (np.abs(a).astype(np.float64).T @ np.abs(b).astype(np.float64)) * 5e-5 + 1e-6  # worst case 3 * 2^-16 per product (bf16 unit roundoff 2^-8)
    assert np.all(np.abs(got - expect) <= bound)
