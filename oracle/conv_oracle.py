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


# ---- weight variance ---------------------------------------------------------------------------------
def compute_variance_weights(basis, feats, neighbors, start_ids, divide_num_neighs):
    """pcconvs/shared/compute_variance_weights.cu:24-170: for every sample the double sum over its neighbors
    (i, j) of (b_i . b_j) (f_i . f_j) [/ n^2], then 1 / mean over the samples.  Restated as the reference
    loops (Gram matrices of the sample's basis rows and feature rows), not through the projected features."""
    n0, _ = _idx(neighbors)
    ends = torch.as_tensor(start_ids).to(torch.int64)
    acc = torch.zeros((ends.shape[0],), dtype=feats.dtype)
    lo = 0
    for m in range(ends.shape[0]):
        hi = int(ends[m])
        if hi > lo:
            b, f = basis[lo:hi], feats[n0[lo:hi]]
            v = ((b @ b.t()) * (f @ f.t())).sum()
            acc[m] = v / float((hi - lo) ** 2) if divide_num_neighs else v
        lo = hi
    return torch.reciprocal(acc.mean())


def kp_conv_weight_var(pts, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, dtype=torch.float64):
    """pcconvs/kpconv.cu:115-135."""
    pts, feats, samples, radii, kernel_pts = _prep(dtype, pts, feats, samples, radii, kernel_pts)
    neighbors = torch.as_tensor(neighbors)
    basis = kernel_pts_basis(pt_diff(pts, samples, neighbors, radii), kernel_pts, float(sigma))
    return compute_variance_weights(basis, feats, neighbors, start_ids, False)


def mc_conv_weight_var(pts, pdf, feats, samples, neighbors, start_ids, radii, axis, bias, dtype=torch.float64):
    """pcconvs/mcconv.cu:146-171."""
    pts, pdf, feats, samples, radii, axis, bias = _prep(dtype, pts, pdf, feats, samples, radii, axis, bias)
    neighbors = torch.as_tensor(neighbors)
    basis = mlp_basis(pt_diff(pts, samples, neighbors, radii), axis, bias, pdf[_idx(neighbors)[0]])
    return compute_variance_weights(basis, feats, neighbors, start_ids, False)


# ---- KPConvN, PCCNN ----------------------------------------------------------------------------------
def kernel_pts_basis_gauss(diffs, kernel_pts, sigma):
    """pcconvs/shared/kernel_pts_basis.cu:72-85: exp(-|kp - d|^2 / (2 sigma^2))."""
    d = kernel_pts.reshape(1, -1, diffs.shape[1]) - diffs.reshape(-1, 1, diffs.shape[1])
    return torch.exp(-((d * d).sum(-1) / (2.0 * sigma * sigma)))


def kernel_pts_basis_gauss_grads(diffs, kernel_pts, sigma, in_grads):
    """pcconvs/shared/kernel_pts_basis.cu:87-111."""
    nk = kernel_pts.shape[0]
    d = kernel_pts.reshape(1, -1, diffs.shape[1]) - diffs.reshape(-1, 1, diffs.shape[1])
    e = torch.exp(-((d * d).sum(-1, keepdim=True) / (2.0 * sigma * sigma)))
    g_kp = -in_grads.reshape(-1, nk, 1) * e * d * (1.0 / (sigma * sigma))
    return (-g_kp).sum(1), g_kp.sum(0)


def _kp_density(pts, pdf, feats, samples, neighbors, radii, kernel_pts, sigma, gauss):
    diffs = pt_diff(pts, samples, neighbors, radii)
    raw = kernel_pts_basis_gauss(diffs, kernel_pts, sigma) if gauss else kernel_pts_basis(diffs, kernel_pts, sigma)
    pdf_n = pdf[_idx(neighbors)[0]].reshape(-1, 1)
    return diffs, raw, pdf_n, raw / pdf_n


def kp_conv_n(pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights, dtype=torch.float64,
              gauss=False):
    """pcconvs/kpconvn.cu:32-68 (gauss=True: pcconvs/pccnn.cu:32-66)."""
    pts, pdf, feats, samples, radii, kernel_pts, weights = _prep(dtype, pts, pdf, feats, samples, radii, kernel_pts, weights)
    neighbors = torch.as_tensor(neighbors)
    _, _, _, basis = _kp_density(pts, pdf, feats, samples, neighbors, radii, kernel_pts, float(sigma), gauss)
    return feat_basis_proj(basis, feats, neighbors, samples.shape[0]).reshape(samples.shape[0], -1) @ weights


def kp_conv_n_grads(pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights, in_grads,
                    dtype=torch.float64):
    """pcconvs/kpconvn.cu:71-130 -> [dW, dFeat, dKernelPts, dPts, dSamples] (no density gradient there)."""
    pts, pdf, feats, samples, radii, kernel_pts, weights, in_grads = _prep(dtype, pts, pdf, feats, samples, radii,
                                                                           kernel_pts, weights, in_grads)
    neighbors = torch.as_tensor(neighbors)
    sigma = float(sigma)
    diffs, _, pdf_n, basis = _kp_density(pts, pdf, feats, samples, neighbors, radii, kernel_pts, sigma, False)
    proj = feat_basis_proj(basis, feats, neighbors, samples.shape[0]).reshape(samples.shape[0], -1)
    d_w = proj.t() @ in_grads
    d_feat, d_basis = feat_basis_proj_grads(basis, feats, neighbors, in_grads @ weights.t())
    d_diff, d_kpts = kernel_pts_basis_grads(diffs, kernel_pts, sigma, d_basis / pdf_n)
    d_pts, d_samples = pt_diff_grads(pts, samples, neighbors, radii, d_diff)
    return [d_w, d_feat, d_kpts, d_pts, d_samples]


def kp_conv_n_weight_var(pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, dtype=torch.float64,
                         gauss=False):
    """pcconvs/kpconvn.cu:133-155 (gauss=True: pcconvs/pccnn.cu:142-165)."""
    pts, pdf, feats, samples, radii, kernel_pts = _prep(dtype, pts, pdf, feats, samples, radii, kernel_pts)
    neighbors = torch.as_tensor(neighbors)
    _, _, _, basis = _kp_density(pts, pdf, feats, samples, neighbors, radii, kernel_pts, float(sigma), gauss)
    return compute_variance_weights(basis, feats, neighbors, start_ids, False)


def pccnn(pts, feats, pdf, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights, dtype=torch.float64):
    """pcconvs/pccnn.cu:32-66 (argument order of the reference: features before the density)."""
    return kp_conv_n(pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights, dtype, gauss=True)


def pccnn_grads(pts, feats, pdf, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights, in_grads,
                dtype=torch.float64):
    """pcconvs/pccnn.cu:69-139 -> [dW, dFeat, dKernelPts, dPdf, dPts, dSamples]."""
    pts, pdf, feats, samples, radii, kernel_pts, weights, in_grads = _prep(dtype, pts, pdf, feats, samples, radii,
                                                                           kernel_pts, weights, in_grads)
    neighbors = torch.as_tensor(neighbors)
    sigma = float(sigma)
    n0 = _idx(neighbors)[0]
    diffs, _, pdf_n, basis = _kp_density(pts, pdf, feats, samples, neighbors, radii, kernel_pts, sigma, True)
    proj = feat_basis_proj(basis, feats, neighbors, samples.shape[0]).reshape(samples.shape[0], -1)
    d_w = proj.t() @ in_grads
    d_feat, d_basis = feat_basis_proj_grads(basis, feats, neighbors, in_grads @ weights.t())
    d_pdf = torch.zeros_like(pdf).index_add_(0, n0, ((-1.0 * basis * d_basis) / pdf_n).sum(1))
    d_diff, d_kpts = kernel_pts_basis_gauss_grads(diffs, kernel_pts, sigma, d_basis / pdf_n)
    d_pts, d_samples = pt_diff_grads(pts, samples, neighbors, radii, d_diff)
    return [d_w, d_feat, d_kpts, d_pdf, d_pts, d_samples]


def pccnn_weight_variance(pts, feats, pdf, samples, neighbors, start_ids, radii, kernel_pts, sigma, dtype=torch.float64):
    return kp_conv_n_weight_var(pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, dtype, gauss=True)


# ---- SPHConv -----------------------------------------------------------------------------------------
def spherical_basis(diffs, radial_bins, azimuz_bins, polar_bins):
    """pcconvs/shared/spherical_basis.cu:24-168: one-hot over (radial, azimuth, polar) bins, bin 0 for offsets
    shorter than 1e-4.  The bin decisions are made in float32, as the reference's kernel makes them."""
    d32 = diffs.to(torch.float32)
    dist = torch.sqrt((d32 * d32).sum(-1))
    az = torch.atan(d32[:, 1] / (d32[:, 0] + 1e-6))
    pol = torch.acos(torch.clamp(d32[:, 2] / (dist + 1e-6), -0.99999, 0.99999))

    def first_bin(v, edges):
        edges = torch.as_tensor(edges, dtype=torch.float32)
        hit = v.reshape(-1, 1) <= edges.reshape(1, -1)
        idx = torch.where(hit.any(1), hit.to(torch.int64).argmax(1), torch.full((v.shape[0],), edges.shape[0] - 1))
        return idx

    nr, na, npol = len(radial_bins), len(azimuz_bins), len(polar_bins)
    ids = first_bin(dist, radial_bins) * na * npol + first_bin(az, azimuz_bins) * npol + first_bin(pol, polar_bins) + 1
    ids = ids * (~(dist < 1e-4)).to(torch.int64)
    basis = torch.zeros((diffs.shape[0], nr * na * npol + 1), dtype=diffs.dtype)
    basis[torch.arange(diffs.shape[0]), ids] = 1.0
    return basis


def _num_neighbors(neighbors, num_samples, dtype):
    return torch.zeros((num_samples,), dtype=dtype).index_add_(0, _idx(neighbors)[1], torch.ones((neighbors.shape[0],), dtype=dtype))


def sph_conv(pts, feats, samples, neighbors, start_ids, radii, radial_bins, azimuz_bins, polar_bins, weights,
             dtype=torch.float64):
    """pcconvs/sphconv.cu:32-72."""
    pts, feats, samples, radii, weights = _prep(dtype, pts, feats, samples, radii, weights)
    neighbors = torch.as_tensor(neighbors)
    basis = spherical_basis(pt_diff(pts, samples, neighbors, radii), radial_bins, azimuz_bins, polar_bins)
    out = feat_basis_proj(basis, feats, neighbors, samples.shape[0]).reshape(samples.shape[0], -1) @ weights
    return out / (_num_neighbors(neighbors, samples.shape[0], out.dtype).reshape(-1, 1) + 1e-6)


def sph_conv_grads(pts, feats, samples, neighbors, start_ids, radii, radial_bins, azimuz_bins, polar_bins, weights,
                   in_grads, dtype=torch.float64):
    """pcconvs/sphconv.cu:75-120 -> [dW, dFeat]."""
    pts, feats, samples, radii, weights, in_grads = _prep(dtype, pts, feats, samples, radii, weights, in_grads)
    neighbors = torch.as_tensor(neighbors)
    g = in_grads / (_num_neighbors(neighbors, samples.shape[0], in_grads.dtype).reshape(-1, 1) + 1e-6)
    basis = spherical_basis(pt_diff(pts, samples, neighbors, radii), radial_bins, azimuz_bins, polar_bins)
    proj = feat_basis_proj(basis, feats, neighbors, samples.shape[0]).reshape(samples.shape[0], -1)
    d_feat, _ = feat_basis_proj_grads(basis, feats, neighbors, g @ weights.t())
    return [proj.t() @ g, d_feat]


def sph_conv_weight_var(pts, feats, samples, neighbors, start_ids, radii, radial_bins, azimuz_bins, polar_bins,
                        dtype=torch.float64):
    """pcconvs/sphconv.cu:123-146 (the only operator that divides by the neighbor count)."""
    pts, feats, samples, radii = _prep(dtype, pts, feats, samples, radii)
    neighbors = torch.as_tensor(neighbors)
    basis = spherical_basis(pt_diff(pts, samples, neighbors, radii), radial_bins, azimuz_bins, polar_bins)
    return compute_variance_weights(basis, feats, neighbors, start_ids, True)


# ---- PointConv ---------------------------------------------------------------------------------------
def point_conv_basis(pts, radii, samples, neighbors, axis, bias, dtype=torch.float64):
    """pcconvs/pointconv.cu:32-51."""
    pts, radii, samples, axis, bias = _prep(dtype, pts, radii, samples, axis, bias)
    return pt_diff(pts, samples, torch.as_tensor(neighbors), radii) @ axis + bias


def point_conv_basis_grads(pts, radii, samples, neighbors, axis, bias, in_grads, dtype=torch.float64):
    """pcconvs/pointconv.cu:54-86 -> [dPts, dSamples, dAxis, dBias]."""
    pts, radii, samples, axis, bias, in_grads = _prep(dtype, pts, radii, samples, axis, bias, in_grads)
    neighbors = torch.as_tensor(neighbors)
    diffs = pt_diff(pts, samples, neighbors, radii)
    d_pts, d_samples = pt_diff_grads(pts, samples, neighbors, radii, in_grads @ axis.t())
    return [d_pts, d_samples, diffs.t() @ in_grads, in_grads.sum(0, keepdim=True)]


def point_conv(basis, feats, neighbors, start_ids, weights, dtype=torch.float64):
    """pcconvs/pointconv.cu:89-103."""
    basis, feats, weights = _prep(dtype, basis, feats, weights)
    m = len(start_ids)
    return feat_basis_proj(basis, feats, torch.as_tensor(neighbors), m).reshape(m, -1) @ weights


def point_conv_grads(basis, feats, neighbors, start_ids, weights, in_grads, dtype=torch.float64):
    """pcconvs/pointconv.cu:106-127 -> [dW, dFeat, dBasis]."""
    basis, feats, weights, in_grads = _prep(dtype, basis, feats, weights, in_grads)
    neighbors = torch.as_tensor(neighbors)
    m = len(start_ids)
    proj = feat_basis_proj(basis, feats, neighbors, m).reshape(m, -1)
    d_feat, d_basis = feat_basis_proj_grads(basis, feats, neighbors, in_grads @ weights.t())
    return [proj.t() @ in_grads, d_feat, d_basis]


def point_conv_weight_var(basis, feats, neighbors, start_ids, dtype=torch.float64):
    """pcconvs/pointconv.cu:130-139."""
    basis, feats = _prep(dtype, basis, feats)
    return compute_variance_weights(basis, feats, torch.as_tensor(neighbors), start_ids, False)
