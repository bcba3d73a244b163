"""Regenerates tests/golden/ref_clouds_32x1000.npy from the reference's own unit-test clouds.

Input: the 32 files unit_test/point_clouds/model{0..31}.xyz of phermosilla/pccnn_lib (100 000
"x y z" lines each).  Each cloud is normalised exactly as unit_test/unit_test.py:43-51 does
(centre of the AABB to the origin, divide by the AABB diagonal, float32 storage) and the first
1000 points are kept, which covers every (batch_size, num_pts) slice the reference's .ini test
configurations take (at most 32 clouds x 1000 points).

Usage: python tests/golden/make_fixtures.py [/path/to/reference]
"""
import os
import sys

import numpy as np


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
        "PCCNN_REFERENCE", os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference")))
    src = os.path.join(ref, "unit_test", "point_clouds")
    out = np.zeros((32, 1000, 3), dtype=np.float32)
    for i in range(32):
        model = np.loadtxt(os.path.join(src, "model%d.xyz" % i))
        max_pt, min_pt = np.amax(model, axis=0), np.amin(model, axis=0)
        center = (max_pt + min_pt) * 0.5
        aabb_size = np.linalg.norm(max_pt - min_pt)
        full = np.zeros((model.shape[0], 3), dtype=np.float32)
        full[:, :] = (model - center) / aabb_size
        out[i] = full[:1000]
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_clouds_32x1000.npy")
    np.save(dst, out)
    print(dst, out.shape, out.dtype)


if __name__ == "__main__":
    main()
