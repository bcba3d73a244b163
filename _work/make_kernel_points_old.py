"""Generates kernel_points.npz: kernel-point dispositions for KPConv in 2, 3 and 4 dimensions
with 8, 16, 32 and 64 points (keys '<dims>_<points>', the naming of the reference's
pccnn_lib/pc/layers/kernel_points/kernel_points.py).

Row 0 is the centre; the other points are spread by minimising a repulsion energy
sum_{i<j} 1/|x_i - x_j| plus a quadratic pull towards the centre (the construction KPConv
uses), from a seeded start, so the file is reproducible.  The tables are not the reference's
numbers: KPConv normalises whatever table it is given, and kernel points are an explicit
operator input, so operator parity does not depend on them.

Usage: python make_kernel_points.py
"""
import os

import numpy as np


def disposition(dims, num_pts, seed, iters=3000):
    rs = np.random.RandomState(seed)
    x = rs.normal(size=(num_pts, dims))
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    x *= rs.uniform(0.3, 1.0, size=(num_pts, 1)) ** (1.0 / dims)
    x[0] = 0.0
    lr = 0.02
    for it in range(iters):
        diff = x[:, None, :] - x[None, :, :]
        dist = np.sqrt((diff ** 2).sum(-1) + 1e-9)
        np.fill_diagonal(dist, np.inf)
        grad = -(diff / dist[..., None] ** 3).sum(1) + 2.0 * 0.5 * num_pts ** (1.0 / dims) * x
        grad[0] = 0.0
        step = lr * (0.999 ** it)
        norm = np.linalg.norm(grad, axis=1, keepdims=True)
        x -= step * grad / np.maximum(norm, 1.0)
    return x


def main():
    out = {}
    for dims in (2, 3, 4):
        for num_pts in (8, 16, 32, 64):
            out["%d_%d" % (dims, num_pts)] = np.round(disposition(dims, num_pts, 100 * dims + num_pts), 6)
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kernel_points.npz")
    np.savez(dst, **out)
    for k, v in out.items():
        n = np.linalg.norm(v, axis=1)
        print(k, v.shape, "min/max radius of the shell points: %.3f %.3f" % (n[1:].min(), n[1:].max()))


if __name__ == "__main__":
    main()
