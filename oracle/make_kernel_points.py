"""Regenerates pccnn_lib_b200/pc/layers/kernel_points/kernel_points.npz and the test fixture
tests/golden/ref_kernel_points_prepared.npz from an installed copy of phermosilla/pccnn_lib.

The KPConv kernel-point dispositions are a table of constants of the reference
(pccnn_lib/pc/layers/kernel_points/kernel_points.py: 12 arrays keyed '<dims>_<points>', row 0 the
centre).  A freshly constructed KPConv layer must start from the same kernel points and sigma as the
reference's layer, so the table is read from the reference by importing that module and stored as
.npz; no source text is copied.  The fixture holds what the reference's constructor makes of every
table (pccnn_lib/pc/layers/KPConv.py:45-57, evaluated here with the reference's own
py_utils/pc_utils.rotate_pc_3d), which tests/test_conv_oracle_pins.py compares with
pccnn_lib_b200.pc.layers.prepare_kernel_points.

Usage: python oracle/make_kernel_points.py [/path/to/reference]
"""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
        "PCCNN_REFERENCE", os.path.normpath(os.path.join(ROOT, "..", "reference")))
    tables = _load(os.path.join(ref, "pccnn_lib", "pc", "layers", "kernel_points", "kernel_points.py"),
                   "_ref_kernel_points").kernel_pts_dict
    pc_utils = _load(os.path.join(ref, "pccnn_lib", "py_utils", "pc_utils.py"), "_ref_pc_utils")
    out = {k: np.asarray(v, dtype=np.float64) for k, v in tables.items()}
    dst = os.path.join(ROOT, "pccnn_lib_b200", "pc", "layers", "kernel_points", "kernel_points.npz")
    np.savez(dst, **out)
    print(dst, sorted(out))

    # What the reference's KPConv constructor registers as kernel_pts_ / sigma_ for every table.
    prepared = {}
    for key, table in out.items():
        pts = table.astype(np.float32)
        dist = np.linalg.norm(pts, axis=-1).astype(np.float32)
        max_dist = np.amax(dist)
        dist = dist / max_dist
        pts = pts / max_dist
        min_distance = np.amin(dist[1:])
        if pts.shape[-1] == 3:
            pts, _ = pc_utils.rotate_pc_3d(np.random.RandomState(15), pts)
        pts = pts.astype(np.float32)
        prepared[key + "_pts"] = pts / (1.0 + min_distance)
        prepared[key + "_sigma"] = np.float64((min_distance * 1.0) / (1.0 + min_distance))
    fix = os.path.join(ROOT, "tests", "golden", "ref_kernel_points_prepared.npz")
    np.savez(fix, **prepared)
    print(fix)


if __name__ == "__main__":
    main()
