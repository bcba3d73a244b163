"""CPU restatement of the KPConv / MCConv operators of phermosilla/pccnn_lib.  TEST INFRASTRUCTURE ONLY.

The reference's convolution ops are ATen compositions around one CUDA kernel pair; this module
restates them with torch on the CPU, stage by stage, citing the reference lines each stage
follows (paths relative to the reference root).  The default dtype is float64 so that the
oracle's own rounding error is far below the tolerances the GPU kernels are held to; pass
``dtype=torch.float32`` to time a like-for-like CPU baseline.

Pinned by tests/test_conv_oracle_pins.py, which replays the NumPy expectations of the
reference's unit_test/test_kpconv.py:60-82 and unit_test/test_mcconv.py:65-91 and checks the
hand-written backward formulas against finite differences of the forward.
"""
import torch


def _idx(neighbors):
    return neighbors[:, 0].to(torch.int64), neighbors[:, 1].to(torch.int64)


def pt_diff(pts, samples, neighbors, radii):
    """pcconvs/shared/pt_diff.cu:27-49: (pts[n0] - samples[n1]) * (1 / radii)."""
    n0, n1 = _idx(neighbors)
    return (pts[n0] - samples[n1]) * torch.reciprocal(radii)


def pt_diff_grads(pts, samples, neighbors, radii, in_grads):
    """pcconvs/shared/pt_diff.cu:51-80."""
    n0, n1 = _idx(neighbors)
    g = in_grads * torch.reciprocal(radii)
    d_pts = torch.zeros_like(pts).index_add_(0, n0, g)
    d_samples = torch.zeros_like(samples).index_add_(0, n1, g) * -1.0
    return d_pts, d_samples


def kernel_pts_basis(diffs, kernel_pts, sigma):
    """pcconvs/shared/kernel_pts_basis.cu:23-39: clamp(1 - |kp - d| / sigma, 0, 1)."""
    d = kernel_pts.reshape(1, -1, diffs.shape[1]) - diffs.reshape(-1, 1, diffs.shape[1])
    dist = torch.sqrt(torch.clamp((d * d).sum(-1), min=0.0))
    return torch.clamp(1.0 - dist / sigma, 0.0, 1.0)


def kernel_pts_basis_grads(diffs, kernel_pts, sigma, in_grads):
    """pcconvs/shared/kernel_pts_basis.cu:41-70 (mask `1 - dist/sigma >= 0`, 1/(dist + 1e-6))."""
    nk = kernel_pts.shape[0]
    d = kernel_pts.reshape(1, -1, diffs.shape[1]) - diffs.reshape(-1, 1, diffs.shape[1])
    dist = torch.sqrt(torch.clamp((d * d).sum(-1), min=0.0))
    result = 1.0 - dist / sigma
    inv = torch.reciprocal((dist + 1e-6).reshape(-1, nk, 1))
    g = in_grads * (result >= 0.0).to(in_grads.dtype)
    g = (-g / sigma).reshape(-1, nk, 1) * inv * d
    return -g.sum(1), g.sum(0)


def mlp_basis(diffs, axis, bias, pdf_n):
    """pcconvs/shared/mlp_basis.cu:27-48 with pDiv = true: leaky_relu(d A + b, 0.2) / pdf."""
    proj = torch.nn.functional.leaky_relu(diffs @ axis + bias, 0.2)
    return proj / pdf_n.reshape(-1, 1)


def mlp_basis_grads(diffs, axis, bias, pdf_n, in_grads):
    """pcconvs/shared/mlp_basis.cu:50-96 with pDiv = true."""
    proj = torch.nn.functional.leaky_relu(diffs @ axis + bias, 0.2)
    d_pdf = ((-1.0 * proj * in_grads) / (pdf_n * pdf_n).reshape(-1, 1)).sum(1)
    cur = in_grads / pdf_n.reshape(-1, 1)
    mask = (proj > 0.0).to(cur.dtype)
    cur = cur * (mask + (1.0 - mask) * 0.2)
    d_bias = cur.sum(0, keepdim=True)
    d_diff = cur @ axis.t()
    d_axis = diffs.t() @ cur
    return d_diff, d_axis, d_bias, d_pdf


def feat_basis_proj(basis, feats, neighbors, num_samples):
    """pcconvs/shared/feat_basis_proj.cu:76-124: P[m, c, k] = sum_t F[n0(t), c] * b[t, k]."""
    n0, n1 = _idx(neighbors)
    outer = feats[n0].unsqueeze(2) * basis.unsqueeze(1)  # [T, Cin, K]
    out = torch.zeros((num_samples, feats.shape[1], basis.shape[1]), dtype=feats.dtype)
    return out.index_add_(0, n1, outer)


def feat_basis_proj_grads(basis, feats, neighbors, in_grads):
    """pcconvs/shared/feat_basis_proj_grads.cu:84-148; in_grads is [M, Cin * K]."""
    n0, n1 = _idx(neighbors)
    g = in_grads.reshape(-1, feats.shape[1], basis.shape[1])[n1]  # [T, Cin, K]
    d_feat = torch.zeros_like(feats).index_add_(0, n0, (g * basis.unsqueeze(1)).sum(2))
    d_basis = (g * feats[n0].unsqueeze(2)).sum(1)
    return d_feat, d_basis


def _prep(dtype, *tensors):
    return [torch.as_tensor(t).to(dtype) if torch.as_tensor(t).is_floating_point() else torch.as_tensor(t)
            for t in tensors]


def kp_conv(pts, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights, dtype=torch.float64):
    """pcconvs/kpconv.cu:32-60."""
    pts, feats, samples, radii, kernel_pts, weights = _prep(dtype, pts, feats, samples, radii, kernel_pts, weights)
    neighbors = torch.as_tensor(neighbors)
    diffs = pt_diff(pts, samples, neighbors, radii)
    basis = kernel_pts_basis(diffs, kernel_pts, float(sigma))
    proj = feat_basis_proj(basis, feats, neighbors, samples.shape[0])
    return proj.reshape(samples.shape[0], -1) @ weights


def kp_conv_grads(pts, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights, in_grads,
                  dtype=torch.float64):
    """pcconvs/kpconv.cu:63-112 -> [dW, dFeat, dKernelPts, dPts, dSamples]."""
    pts, feats, samples, radii, kernel_pts, weights, in_grads = _prep(dtype, pts, feats, samples, radii, kernel_pts,
                                                                      weights, in_grads)
    neighbors = torch.as_tensor(neighbors)
    sigma = float(sigma)
    diffs = pt_diff(pts, samples, neighbors, radii)
    basis = kernel_pts_basis(diffs, kernel_pts, sigma)
    proj = feat_basis_proj(basis, feats, neighbors, samples.shape[0]).reshape(samples.shape[0], -1)
    d_w = proj.t() @ in_grads
    d_proj = in_grads @ weights.t()
    d_feat, d_basis = feat_basis_proj_grads(basis, feats, neighbors, d_proj)
    d_diff, d_kpts = kernel_pts_basis_grads(diffs, kernel_pts, sigma, d_basis)
    d_pts, d_samples = pt_diff_grads(pts, samples, neighbors, radii, d_diff)
    return [d_w, d_feat, d_kpts, d_pts, d_samples]


def mc_conv(pts, pdf, feats, samples, neighbors, start_ids, radii, axis, bias, weights, dtype=torch.float64):
    """pcconvs/mcconv.cu:32-71 (weights [numMLPs, H * Cin, Cout / numMLPs])."""
    pts, pdf, feats, samples, radii, axis, bias, weights = _prep(dtype, pts, pdf, feats, samples, radii, axis, bias,
                                                                 weights)
    neighbors = torch.as_tensor(neighbors)
    n_mlps, m = weights.shape[0], samples.shape[0]
    diffs = pt_diff(pts, samples, neighbors, radii)
    basis = mlp_basis(diffs, axis, bias, pdf[_idx(neighbors)[0]])
    proj = feat_basis_proj(basis, feats, neighbors, m).reshape(m, n_mlps, -1).transpose(0, 1)
    return torch.matmul(proj, weights).transpose(0, 1).reshape(m, -1)


def mc_conv_grads(pts, pdf, feats, samples, neighbors, start_ids, radii, axis, bias, weights, in_grads,
                  dtype=torch.float64):
    """pcconvs/mcconv.cu:73-143 -> [dW, dFeat, dAxis, dBias, dPdf, dPts, dSamples]."""
    pts, pdf, feats, samples, radii, axis, bias, weights, in_grads = _prep(
        dtype, pts, pdf, feats, samples, radii, axis, bias, weights, in_grads)
    neighbors = torch.as_tensor(neighbors)
    n_mlps, m = weights.shape[0], samples.shape[0]
    n0 = _idx(neighbors)[0]
    g = in_grads.reshape(m, n_mlps, -1).transpose(0, 1)
    diffs = pt_diff(pts, samples, neighbors, radii)
    pdf_n = pdf[n0]
    basis = mlp_basis(diffs, axis, bias, pdf_n)
    proj = feat_basis_proj(basis, feats, neighbors, m).reshape(m, n_mlps, -1)
    d_w = torch.matmul(proj.transpose(0, 1).transpose(1, 2), g)
    d_proj = torch.matmul(g, weights.transpose(1, 2)).transpose(0, 1).reshape(m, -1)
    d_feat, d_basis = feat_basis_proj_grads(basis, feats, neighbors, d_proj)
    d_diff, d_axis, d_bias, d_pdf_t = mlp_basis_grads(diffs, axis, bias, pdf_n, d_basis)
    d_pdf = torch.zeros_like(pdf).index_add_(0, n0, d_pdf_t)
    d_pts, d_samples = pt_diff_grads(pts, samples, neighbors, radii, d_diff)
    return [d_w, d_feat, d_axis, d_bias, d_pdf, d_pts, d_samples]
