"""NumPy front end of the CPU oracle (oracle/pccnn_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and the CPU-baseline legs of bench.py may import this
module; the pccnn_lib_b200 package never does.  Function names and argument order follow the
reference's pccnn_lib_ops module (pccnn_lib_ops/ops_list.cpp:27-43 of phermosilla/pccnn_lib) so
that a parity test reads `oracle.f(args)` against `ops.f(args)`.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_build", "libpccnn_oracle.so")


def build(force=False):
    src = os.path.join(HERE, "pccnn_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE] + (["-B"] if force else []), check=True, capture_output=True)
    return LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.orc_find_neighbors_count.restype = ctypes.c_int64
        _lib.orc_poisson_disk_sampling.restype = ctypes.c_int64
    return _lib


def set_threads(n):
    """Asks the OpenMP runtime of the oracle for n threads; returns how many it will use."""
    return int(lib().orc_set_threads(int(n)))


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


_I64 = ctypes.c_int64
_INT = ctypes.c_int


def bounding_box(pts, batch_ids, num_batches):
    pts, batch_ids = _f32(pts), _i32(batch_ids)
    n, d = pts.shape
    mn = np.empty((num_batches, d), np.float32)
    mx = np.empty((num_batches, d), np.float32)
    lib().orc_bounding_box(_INT(d), _I64(n), _ptr(pts), _ptr(batch_ids), _I64(num_batches), _ptr(mn), _ptr(mx))
    return mn, mx


def grid_num_cells(aabb_min, aabb_max, cell_size):
    aabb_min, aabb_max, cell_size = _f32(aabb_min), _f32(aabb_max), _f32(cell_size)
    b, d = aabb_min.shape
    out = np.empty((d,), np.int32)
    lib().orc_grid_num_cells(_INT(d), _I64(b), _ptr(aabb_min), _ptr(aabb_max), _ptr(cell_size), _ptr(out))
    return out


def compute_keys(pts, batch_ids, aabb_min, grid_size, cell_size):
    pts, batch_ids, aabb_min = _f32(pts), _i32(batch_ids), _f32(aabb_min)
    grid_size, cell_size = _i32(grid_size), _f32(cell_size)
    n, d = pts.shape
    out = np.empty((n,), np.int64)
    lib().orc_compute_keys(_INT(d), _I64(n), _ptr(pts), _ptr(batch_ids), _ptr(aabb_min), _ptr(grid_size),
                           _ptr(cell_size), _ptr(out))
    return out


def stable_argsort(keys):
    keys = _i64(keys)
    out = np.empty_like(keys)
    lib().orc_stable_argsort(_I64(keys.shape[0]), _ptr(keys), _ptr(out))
    return out


def build_grid_ds(sorted_keys, grid_size, out_shape):
    sorted_keys, grid_size = _i64(sorted_keys), _i32(grid_size)
    out = np.empty(tuple(int(v) for v in out_shape), np.int32)
    entries = int(out_shape[0]) * int(out_shape[1]) * int(out_shape[2])
    lib().orc_build_grid_ds(_INT(grid_size.shape[0]), _I64(sorted_keys.shape[0]), _ptr(sorted_keys),
                            _ptr(grid_size), _I64(entries), _ptr(out))
    return out


def find_neighbors(pts, pt_keys, samples, sample_keys, grid_ds, grid_size, radii, max_neighbors):
    pts, pt_keys, samples, sample_keys = _f32(pts), _i64(pt_keys), _f32(samples), _i64(sample_keys)
    grid_ds, grid_size, radii = _i32(grid_ds), _i32(grid_size), _f32(radii)
    n, d = pts.shape
    m = samples.shape[0]
    counts = np.empty((m,), np.int32)
    start_ids = np.empty((m,), np.int32)
    common = (_INT(d), _I64(n), _ptr(pts), _ptr(pt_keys), _I64(m), _ptr(samples), _ptr(sample_keys),
              _ptr(grid_ds), _ptr(grid_size), _ptr(radii), ctypes.c_int32(int(max_neighbors)))
    total = lib().orc_find_neighbors_count(*common, _ptr(counts), _ptr(start_ids))
    neighbors = np.empty((total, 2), np.int32)
    lib().orc_find_neighbors_store(*common, _ptr(counts), _ptr(start_ids), _ptr(neighbors))
    return neighbors, start_ids


def compute_pdf(manifold_dims, bandwidth, pts, neighbors, start_ids):
    bandwidth, pts, neighbors, start_ids = _f32(bandwidth), _f32(pts), _i32(neighbors), _i32(start_ids)
    n, d = pts.shape
    out = np.empty((n,), np.float32)
    lib().orc_compute_pdf(_INT(d), _INT(int(manifold_dims)), _ptr(bandwidth), _I64(n), _ptr(pts), _ptr(neighbors),
                          _ptr(start_ids), _ptr(out))
    return out


def compute_pdf_grads(manifold_dims, bandwidth, pts, neighbors, start_ids, in_grads):
    bandwidth, pts, neighbors, start_ids = _f32(bandwidth), _f32(pts), _i32(neighbors), _i32(start_ids)
    in_grads = _f32(in_grads)
    n, d = pts.shape
    out = np.empty((n, d), np.float64)
    lib().orc_compute_pdf_grads(_INT(d), _INT(int(manifold_dims)), _ptr(bandwidth), _I64(n), _ptr(pts),
                                _ptr(neighbors), _ptr(start_ids), _ptr(in_grads), _ptr(out))
    return out


def poisson_disk_sampling(sorted_keys, neighbors, start_ids, grid_size):
    sorted_keys, neighbors, start_ids, grid_size = _i64(sorted_keys), _i32(neighbors), _i32(start_ids), _i32(grid_size)
    n = sorted_keys.shape[0]
    out = np.empty((n,), np.int64)
    k = lib().orc_poisson_disk_sampling(_INT(grid_size.shape[0]), _I64(n), _ptr(sorted_keys), _ptr(neighbors),
                                        _ptr(start_ids), _ptr(grid_size), _ptr(out))
    return out[:k].reshape(-1, 1)


# ---- pipelines built from the pieces above (the caller-side code of the reference) ------------
def build_grid(pts, batch_ids, num_batches, cell_size):
    """BoundingBox + Grid.compute_cell_ids + Grid.build_ds (pccnn_lib/pc/BoundingBox.py:17-18,
    pc/Grid.py:27-28,36-72 of the reference) with a stable sort.  Returns a dict."""
    pts, batch_ids, cell_size = _f32(pts), _i32(batch_ids), _f32(cell_size)
    mn, mx = bounding_box(pts, batch_ids, num_batches)
    nc = grid_num_cells(mn, mx, cell_size)
    keys = compute_keys(pts, batch_ids, mn, nc, cell_size)
    ids = stable_argsort(keys)
    skeys = keys[ids]
    ds = build_grid_ds(skeys, nc, [num_batches, nc[0], nc[1], 2])
    return dict(aabb_min=mn, aabb_max=mx, num_cells=nc, keys=keys, sorted_ids=ids, sorted_keys=skeys,
                sorted_pts=pts[ids], grid_ds=ds, cell_size=cell_size)


def brute_force_neighbors(pts, batch_ids, samples, sample_batch_ids, radius):
    """O(N*M) NumPy search exactly as unit_test/test_find_neighs.py:55-67 of the reference does it
    (float32 coordinates, sqrt of the summed squares, strict <).  Returns per-sample index arrays."""
    pts, samples = _f32(pts), _f32(samples)
    out = []
    for m in range(samples.shape[0]):
        diff = pts - samples[m].reshape(1, -1)
        dist = np.sqrt(np.sum(diff * diff, axis=-1))
        mask = np.logical_and(dist < radius, batch_ids == sample_batch_ids[m])
        out.append(np.where(mask)[0])
    return out
