import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")

# Every operator that takes a neighbor list checks it first in the tests (pccnn_lib_b200.ops.validate_neighbors).
os.environ.setdefault("PCCNN_VALIDATE_NEIGHBORS", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def ref_clouds():
    """First 1000 points of the reference's 32 unit-test clouds, normalised as its harness does."""
    return np.load(os.path.join(GOLDEN, "ref_clouds_32x1000.npy"))


def ref_case(clouds, batch_size, num_pts, num_dims):
    """Point / batch-id arrays sliced exactly as the reference's tests slice their dataset
    (e.g. unit_test/test_find_neighs.py:20-32 of phermosilla/pccnn_lib)."""
    pts = clouds[0:batch_size, 0:num_pts, :].reshape((-1, 3))
    if num_dims < 3:
        pts = pts[:, 0:num_dims]
    elif num_dims > 3:
        pts = np.concatenate([pts[:, 0:3], pts[:, 0:num_dims - 3]], axis=-1)
    batch_ids = np.repeat(np.arange(batch_size).reshape((batch_size, 1)), num_pts, 1).reshape((-1)).astype(np.int32)
    return np.ascontiguousarray(pts, dtype=np.float32), batch_ids


def synthetic_case(seed, batch_size, num_pts, num_dims, ragged=True):
    """Seeded clouds with different sizes and extents per cloud."""
    rs = np.random.RandomState(seed)
    pts, ids = [], []
    for b in range(batch_size):
        n = max(1, int(num_pts * rs.uniform(0.5, 1.0))) if ragged else num_pts
        scale = rs.uniform(0.5, 1.5, size=(1, num_dims))
        pts.append((rs.rand(n, num_dims) * scale + rs.uniform(-1, 1, size=(1, num_dims))).astype(np.float32))
        ids.append(np.full((n,), b, np.int32))
    return np.concatenate(pts, 0), np.concatenate(ids, 0)
