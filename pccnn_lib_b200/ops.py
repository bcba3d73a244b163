"""Operator module with the call signatures of the reference's ``pccnn_lib_ops`` extension.

Each function mirrors one ``m.def`` of pccnn_lib_ops/ops_list.cpp:27-43 of phermosilla/pccnn_lib
(same argument order, meaning, dtypes and output shapes) and forwards to the C ABI of
libpccnn_b200.so with raw device pointers on the current CUDA stream.  Outputs are allocated
with torch so they live in the caller's caching allocator.  Tensors must be CUDA tensors:
there is no CPU path.
"""
import contextlib
import ctypes
import os

import torch

from . import _capi

_lib = _capi.lib


def set_conv_path(path):
    """Which kernels do the per-pair work of the convolutions: "tensor" (default: tcgen05 pair kernels for 3-D points
    with at least 32 input channels, CUDA-core kernels otherwise) or "simt" (CUDA-core kernels everywhere).  The
    environment variable PCCNN_CONV_PATH selects it at import."""
    _capi.check(_lib.pccnn_conv_set_path({"tensor": 0, "simt": 1}[path]), "conv_set_path")


set_conv_path(os.environ.get("PCCNN_CONV_PATH", "tensor"))


# ---- argument plumbing -----------------------------------------------------------------------
def _need(t, name, dtype, ndim=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError("%s must be a torch.Tensor" % name)
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor (pccnn_lib_b200 has no CPU path)" % name)
    if t.dtype != dtype:
        raise RuntimeError("%s must have dtype %s, got %s" % (name, dtype, t.dtype))
    if ndim is not None and t.dim() != ndim:
        raise RuntimeError("%s must have %d dimensions, got %d" % (name, ndim, t.dim()))
    return t if t.is_contiguous() else t.contiguous()


def _p(t):
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


_SAME_DEVICE = contextlib.nullcontext()


def _on(device):
    """Makes `device` current for the call; free when it already is (the usual case)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _SAME_DEVICE
    return torch.cuda.device(device)


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)


def _dims(pts, name="pts"):
    d = pts.shape[1]
    if d < 2 or d > 6:
        raise RuntimeError("%s has %d dimensions; supported range is [2, 6]" % (name, d))
    return d


# ---- failure reporting and input validation -----------------------------------------------------
def check_status(synchronize=True):
    """Raises RuntimeError if a tensor-core kernel of an earlier convolution call gave up on one of its bounded
    waits (its outputs are then incomplete).  With `synchronize` the current stream is waited for first, so
    nothing enqueued so far can be missed; without it only failures that already reached the host are seen.
    The convolution operators make the cheap check themselves at every call, so a failure surfaces at the next
    convolution at the latest.  No counterpart in the reference, which checks nothing."""
    _capi.check(_lib.pccnn_check_status(1 if synchronize else 0, _stream()), "check_status")


def validate_neighbors(neighbors, start_ids, num_pts):
    """Checks a neighbor list on the device (indices in range, rows grouped by sample, end offsets monotone and
    ending at T) and raises RuntimeError naming the first bad row instead of letting a later kernel read out of
    bounds.  Synchronises.  Runs automatically in front of every operator that takes a list when the environment
    variable PCCNN_VALIDATE_NEIGHBORS is set to 1."""
    neighbors = _need(neighbors, "neighbors", torch.int32, 2)
    start_ids = _need(start_ids, "start_ids", torch.int32, 1)
    if neighbors.shape[1] != 2:
        raise RuntimeError("neighbors must be [T, 2]")
    with _on(start_ids.device):
        ws = _workspace(_lib.pccnn_validate_neighbors_workspace_bytes(), start_ids.device)
        _capi.check(_lib.pccnn_validate_neighbors(int(num_pts), start_ids.shape[0], _p(neighbors), _p(start_ids),
                                                  neighbors.shape[0], ws.data_ptr(), ws.numel(), _stream()),
                    "validate_neighbors")


def _maybe_validate(neighbors, start_ids, num_pts):
    if os.environ.get("PCCNN_VALIDATE_NEIGHBORS", "0") == "1":
        validate_neighbors(neighbors, start_ids, num_pts)


# ---- grid front end --------------------------------------------------------------------------
def bounding_box(pts, batch_ids, num_batches):
    """Per-cloud (min - 1e-6, max + 1e-6); pccnn_lib/pc/BoundingBox.py:17-18 of the reference."""
    pts = _need(pts, "pts", torch.float32, 2)
    batch_ids = _need(batch_ids, "batch_ids", torch.int32, 1)
    d = _dims(pts)
    b = int(num_batches)
    mn = torch.empty((b, d), dtype=torch.float32, device=pts.device)
    mx = torch.empty((b, d), dtype=torch.float32, device=pts.device)
    with _on(pts.device):
        _capi.check(_lib.pccnn_bounding_box(d, pts.shape[0], _p(pts), _p(batch_ids), b, _p(mn), _p(mx),
                                            _stream()), "bounding_box")
    return mn, mx


def grid_num_cells(aabb_min, aabb_max, cell_size):
    """Cells per dimension shared by all clouds; pccnn_lib/pc/Grid.py:27-28 of the reference."""
    aabb_min = _need(aabb_min, "aabb_min", torch.float32, 2)
    aabb_max = _need(aabb_max, "aabb_max", torch.float32, 2)
    cell_size = _need(cell_size, "cell_size", torch.float32, 1)
    d = aabb_min.shape[1]
    out = torch.empty((d,), dtype=torch.int32, device=aabb_min.device)
    with _on(aabb_min.device):
        _capi.check(_lib.pccnn_grid_num_cells(d, aabb_min.shape[0], _p(aabb_min), _p(aabb_max), _p(cell_size),
                                              _p(out), _stream()), "grid_num_cells")
    return out


def compute_keys(pts, batch_ids, aabb_min, grid_size, cell_size):
    """int64 grid key per point; compute_keys() of compute_keys/compute_keys.cu:78-128."""
    pts = _need(pts, "pts", torch.float32, 2)
    batch_ids = _need(batch_ids, "batch_ids", torch.int32, 1)
    aabb_min = _need(aabb_min, "aabb_min", torch.float32, 2)
    grid_size = _need(grid_size, "grid_size", torch.int32, 1)
    cell_size = _need(cell_size, "cell_size", torch.float32, 1)
    d = _dims(pts)
    if grid_size.numel() != d or cell_size.numel() != d or aabb_min.shape[1] != d:
        raise RuntimeError("grid_size, cell_size and aabb_min must match the point dimension %d" % d)
    if batch_ids.shape[0] != pts.shape[0]:
        raise RuntimeError("batch_ids and pts disagree on the number of points")
    out = torch.empty((pts.shape[0],), dtype=torch.int64, device=pts.device)
    with _on(pts.device):
        _capi.check(_lib.pccnn_compute_keys(d, pts.shape[0], _p(pts), _p(batch_ids), _p(aabb_min),
                                            _p(grid_size), _p(cell_size), _p(out), _stream()), "compute_keys")
    return out


def sort_keys(keys, key_bits=64, pts=None):
    """Stable sort of the keys -> (sorted_keys, sorted_ids[, sorted_pts]).

    Replaces torch.argsort of pccnn_lib/pc/Grid.py:52 and the index_select gathers that follow
    it (Grid.py:68-70, Neighborhood.py:27-32).  Ties keep ascending original index.
    """
    keys = _need(keys, "keys", torch.int64, 1)
    n = keys.shape[0]
    sorted_keys = torch.empty_like(keys)
    sorted_ids = torch.empty_like(keys)
    d, sorted_pts = 0, None
    if pts is not None:
        pts = _need(pts, "pts", torch.float32, 2)
        d = _dims(pts)
        sorted_pts = torch.empty_like(pts)
    with _on(keys.device):
        nbytes = _lib.pccnn_sort_keys_workspace_bytes(n)
        ws = _workspace(nbytes, keys.device)
        _capi.check(_lib.pccnn_sort_keys(n, _p(keys), int(key_bits), _p(sorted_keys), _p(sorted_ids), d, _p(pts),
                                         _p(sorted_pts), ws.data_ptr(), ws.numel(), _stream()), "sort_keys")
    if pts is None:
        return sorted_keys, sorted_ids
    return sorted_keys, sorted_ids, sorted_pts


def grid_front_end(pts, batch_ids, num_batches, cell_size):
    """Bounding boxes, cells per axis, keys, stable sort, sorted copies and the cell table of one
    point set in two library calls and one host synchronisation.

    The caller-side sequence BoundingBox / Grid.__init__ / compute_cell_ids / build_ds of the
    reference (pccnn_lib/pc/BoundingBox.py:10-18, pc/Grid.py:10-72) as one operator.  Returns a dict
    with aabb_min, aabb_max, num_cells (device int32), num_cells_host (list), keys, sorted_keys,
    sorted_ids, sorted_pts, grid_ds.
    """
    pts = _need(pts, "pts", torch.float32, 2)
    batch_ids = _need(batch_ids, "batch_ids", torch.int32, 1)
    cell_size = _need(cell_size, "cell_size", torch.float32, 1)
    d, n, b, dev = _dims(pts), pts.shape[0], int(num_batches), pts.device
    if cell_size.numel() != d or batch_ids.shape[0] != n:
        raise RuntimeError("cell_size / batch_ids do not match pts")
    if n == 0 or b <= 0:
        raise RuntimeError("grid_front_end: needs at least one point and one cloud (an empty set has no bounding box)")
    mn = torch.empty((b, d), dtype=torch.float32, device=dev)
    mx = torch.empty((b, d), dtype=torch.float32, device=dev)
    cells = torch.empty((d,), dtype=torch.int32, device=dev)
    keys = torch.empty((n,), dtype=torch.int64, device=dev)
    sorted_keys, sorted_ids, sorted_pts = torch.empty_like(keys), torch.empty_like(keys), torch.empty_like(pts)
    host_cells = (ctypes.c_int32 * d)()
    with _on(dev):
        stream = _stream()
        ws = _workspace(_lib.pccnn_grid_front_end_workspace_bytes(n), dev)
        _capi.check(_lib.pccnn_grid_front_end(d, n, _p(pts), _p(batch_ids), b, _p(cell_size), _p(mn), _p(mx), _p(cells),
                                              host_cells, _p(keys), _p(sorted_keys), _p(sorted_ids), _p(sorted_pts),
                                              ws.data_ptr(), ws.numel(), stream), "grid_front_end")
        num_cells_host = [int(v) for v in host_cells]
        grid_ds = torch.empty((b, num_cells_host[0], num_cells_host[1], 2), dtype=torch.int32, device=dev)
        _capi.check(_lib.pccnn_build_grid_ds(d, n, _p(sorted_keys), _p(cells), grid_ds.numel() // 2, _p(grid_ds),
                                             stream), "build_grid_ds")
    return dict(aabb_min=mn, aabb_max=mx, num_cells=cells, num_cells_host=num_cells_host, keys=keys,
                sorted_keys=sorted_keys, sorted_ids=sorted_ids, sorted_pts=sorted_pts, grid_ds=grid_ds)


def build_grid_ds(keys, grid_size, out_shape):
    """[B, nc0, nc1, 2] int32 cell-range table; build_grid_ds() of build_grid/build_grid_ds.cu:72-114."""
    keys = _need(keys, "keys", torch.int64, 1)
    grid_size = _need(grid_size, "grid_size", torch.int32, 1)
    shape = [int(v) for v in out_shape]
    if len(shape) != 4 or shape[3] != 2:
        raise RuntimeError("out_shape must be [batch, cells0, cells1, 2], got %s" % (shape,))
    d = grid_size.numel()
    out = torch.empty(shape, dtype=torch.int32, device=keys.device)
    entries = shape[0] * shape[1] * shape[2]
    with _on(keys.device):
        _capi.check(_lib.pccnn_build_grid_ds(d, keys.shape[0], _p(keys), _p(grid_size), entries, _p(out),
                                             _stream()), "build_grid_ds")
    return out


# ---- neighbor search -------------------------------------------------------------------------
class _NeighborSearch(object):
    """State carried from the count call to the store call of one neighbor search."""
    __slots__ = ("common", "start_ids", "total", "workspace", "device", "pt_index_map", "keep")


def find_neighbors_count(pts, pt_keys, samples, sample_keys, grid_ds, grid_size, radii, max_neighbors,
                         pt_index_map=None, workspace_bytes=None, key_bits=0):
    """First half of find_neighbors: counts, scans and learns T (one host synchronisation).
    Returns the state object to hand to find_neighbors_store.  `workspace_bytes` overrides the
    recommended scratch size (never below the library's minimum); a smaller scratch only makes
    the store pass repeat more distance tests.  `key_bits` (0 = unknown): how many low bits of the keys
    can be set, which shortens the ordering of samples that are not the sorted points themselves."""
    pts = _need(pts, "pts", torch.float32, 2)
    pt_keys = _need(pt_keys, "pt_keys", torch.int64, 1)
    samples = _need(samples, "samples", torch.float32, 2)
    sample_keys = _need(sample_keys, "sample_keys", torch.int64, 1)
    grid_ds = _need(grid_ds, "grid_ds", torch.int32)
    grid_size = _need(grid_size, "grid_size", torch.int32, 1)
    radii = _need(radii, "radii", torch.float32, 1)
    if pt_index_map is not None:
        pt_index_map = _need(pt_index_map, "pt_index_map", torch.int64, 1)
    d = _dims(pts)
    if samples.shape[1] != d or grid_size.numel() != d or radii.numel() != d:
        raise RuntimeError("samples, grid_size and radii must match the point dimension %d" % d)
    n, m = pts.shape[0], samples.shape[0]
    if pt_keys.shape[0] != n or sample_keys.shape[0] != m:
        raise RuntimeError("keys and coordinates disagree on the number of rows")
    st = _NeighborSearch()
    st.device = pts.device
    st.pt_index_map = pt_index_map
    st.keep = (pts, pt_keys, samples, sample_keys, grid_ds, grid_size, radii)  # keep the inputs alive
    st.start_ids = torch.empty((m,), dtype=torch.int32, device=pts.device)
    total = ctypes.c_int64(0)
    with _on(pts.device):
        nbytes = _lib.pccnn_find_neighbors_workspace_bytes(d, m)
        if workspace_bytes is not None:
            nbytes = max(int(workspace_bytes), _lib.pccnn_find_neighbors_min_workspace_bytes(d, m))
        st.workspace = _workspace(nbytes, pts.device)
        st.common = (d, n, _p(pts), _p(pt_keys), m, _p(samples), _p(sample_keys), _p(grid_ds), _p(grid_size),
                     _p(radii), int(max_neighbors))
        _capi.check(_lib.pccnn_find_neighbors_count(*st.common, int(key_bits), _p(st.start_ids), ctypes.byref(total),
                                                    st.workspace.data_ptr(), st.workspace.numel(), _stream()),
                    "find_neighbors (count)")
    st.total = total.value
    return st


def find_neighbors_store(st):
    """Second half of find_neighbors: allocates the [T, 2] list and fills it."""
    neighbors = torch.empty((st.total, 2), dtype=torch.int32, device=st.device)
    with _on(st.device):
        _capi.check(_lib.pccnn_find_neighbors_store(*st.common, _p(st.start_ids), _p(st.pt_index_map), _p(neighbors),
                                                    st.workspace.data_ptr(), st.workspace.numel(), _stream()),
                    "find_neighbors (store)")
    return [neighbors, st.start_ids]


def find_neighbors(pts, pt_keys, samples, sample_keys, grid_ds, grid_size, radii, max_neighbors,
                   pt_index_map=None, workspace_bytes=None, key_bits=0):
    """Radius search -> [neighbors [T, 2] int32, start_ids [M] int32 (inclusive ends)].

    find_neighbors() of find_neighbors/find_neighbors.cu:27-66 of the reference.  `pts` and
    `pt_keys` are in sorted order; row.x indexes that array unless `pt_index_map` (an
    extension: the sorted_ids permutation) is given, in which case row.x is mapped through it
    as pccnn_lib/pc/Neighborhood.py:47-53 does afterwards.
    """
    return find_neighbors_store(find_neighbors_count(pts, pt_keys, samples, sample_keys, grid_ds, grid_size, radii,
                                                     max_neighbors, pt_index_map, workspace_bytes, key_bits))


# ---- kernel density estimation ---------------------------------------------------------------
def _pdf_args(bandwidth, pts, neighbors, start_ids):
    bandwidth = _need(bandwidth, "bandwidth", torch.float32, 1)
    pts = _need(pts, "pts", torch.float32, 2)
    neighbors = _need(neighbors, "neighbors", torch.int32, 2)
    start_ids = _need(start_ids, "start_ids", torch.int32, 1)
    d = _dims(pts)
    if bandwidth.numel() != d:
        raise RuntimeError("bandwidth must have %d entries" % d)
    if start_ids.shape[0] != pts.shape[0]:
        raise RuntimeError("start_ids must have one entry per point")
    if neighbors.shape[1] != 2:
        raise RuntimeError("neighbors must be [T, 2]")
    _maybe_validate(neighbors, start_ids, pts.shape[0])
    return bandwidth, pts, neighbors, start_ids, d


def compute_pdf(manifold_dims, bandwidth, pts, neighbors, start_ids):
    """Unnormalised KDE per point; compute_pdf() of compute_pdf/compute_pdf.cu:153-203."""
    bandwidth, pts, neighbors, start_ids, d = _pdf_args(bandwidth, pts, neighbors, start_ids)
    out = torch.empty((pts.shape[0],), dtype=torch.float32, device=pts.device)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_compute_pdf_workspace_bytes(d, pts.shape[0]), pts.device)
        _capi.check(_lib.pccnn_compute_pdf(d, int(manifold_dims), _p(bandwidth), pts.shape[0], _p(pts),
                                           _p(neighbors), _p(start_ids), _p(out), ws.data_ptr(), ws.numel(), _stream()),
                    "compute_pdf")
    return out


def compute_pdf_grads(manifold_dims, bandwidth, pts, neighbors, start_ids, in_grads, full_self_neighborhood=False):
    """Point gradients of the KDE; compute_pdf_grads() of compute_pdf/compute_pdf.cu:206-257.

    `full_self_neighborhood` (an extension): the caller vouches that the list is the uncapped neighborhood of the
    points in themselves, so that every pair appears in both rows; the gradient is then one pass over each point's
    own row without reductions into other rows."""
    bandwidth, pts, neighbors, start_ids, d = _pdf_args(bandwidth, pts, neighbors, start_ids)
    in_grads = _need(in_grads, "in_grads", torch.float32, 1)
    if in_grads.shape[0] != pts.shape[0]:
        raise RuntimeError("in_grads must have one entry per point")
    out = torch.empty_like(pts)
    with _on(pts.device):
        if full_self_neighborhood:
            ws = _workspace(_lib.pccnn_compute_pdf_workspace_bytes(d, pts.shape[0]), pts.device)
            _capi.check(_lib.pccnn_compute_pdf_grads_symmetric(d, int(manifold_dims), _p(bandwidth), pts.shape[0],
                                                               _p(pts), _p(neighbors), _p(start_ids), _p(in_grads),
                                                               _p(out), ws.data_ptr(), ws.numel(), _stream()),
                        "compute_pdf_grads (full self-neighborhood)")
        else:
            _capi.check(_lib.pccnn_compute_pdf_grads(d, int(manifold_dims), _p(bandwidth), pts.shape[0], _p(pts),
                                                     _p(neighbors), _p(start_ids), _p(in_grads), _p(out), _stream()),
                        "compute_pdf_grads")
    return out


# ---- Poisson-disk sampling -------------------------------------------------------------------
def poisson_disk_sampling(sorted_keys, neighbors, start_ids, grid_size):
    """Selected positions [k, 1] int64 (ascending); poisson_disk_sampling() of
    poisson_disk_sampling/poisson_disk_sampling.cu:110-196 of the reference."""
    sorted_keys = _need(sorted_keys, "sorted_keys", torch.int64, 1)
    neighbors = _need(neighbors, "neighbors", torch.int32, 2)
    start_ids = _need(start_ids, "start_ids", torch.int32, 1)
    grid_size = _need(grid_size, "grid_size", torch.int32, 1)
    n = sorted_keys.shape[0]
    d = grid_size.numel()
    if start_ids.shape[0] != n:
        raise RuntimeError("start_ids must have one entry per point")
    _maybe_validate(neighbors, start_ids, n)
    selected = torch.empty((n,), dtype=torch.int64, device=sorted_keys.device)
    count = ctypes.c_int64(0)
    with _on(sorted_keys.device):
        ws = _workspace(_lib.pccnn_poisson_disk_sampling_workspace_bytes(n), sorted_keys.device)
        _capi.check(_lib.pccnn_poisson_disk_sampling(d, n, _p(sorted_keys), _p(neighbors), _p(start_ids),
                                                     _p(grid_size), _p(selected), ctypes.byref(count),
                                                     ws.data_ptr(), ws.numel(), _stream()),
                    "poisson_disk_sampling")
    return selected[:count.value].reshape(-1, 1)


def poisson_disk_sampling_grid(sorted_pts, sorted_keys, grid_ds, grid_size, radii):
    """The selection of poisson_disk_sampling on the full self-neighborhood (radius = cell size)
    without building that neighborhood: [k, 1] int64 ascending sorted positions.  Stands for the
    pair find_neighbors + poisson_disk_sampling of pccnn_lib/pc/PointPooling.py:39-69."""
    sorted_pts = _need(sorted_pts, "sorted_pts", torch.float32, 2)
    sorted_keys = _need(sorted_keys, "sorted_keys", torch.int64, 1)
    grid_ds = _need(grid_ds, "grid_ds", torch.int32, 4)
    grid_size = _need(grid_size, "grid_size", torch.int32, 1)
    radii = _need(radii, "radii", torch.float32, 1)
    d, n = _dims(sorted_pts), sorted_pts.shape[0]
    if sorted_keys.shape[0] != n or grid_size.numel() != d or radii.numel() != d:
        raise RuntimeError("poisson_disk_sampling_grid: sizes of keys / grid_size / radii do not match the points")
    selected = torch.empty((n,), dtype=torch.int64, device=sorted_pts.device)
    count = ctypes.c_int64(0)
    with _on(sorted_pts.device):
        ws = _workspace(_lib.pccnn_poisson_disk_sampling_grid_workspace_bytes(n), sorted_pts.device)
        _capi.check(_lib.pccnn_poisson_disk_sampling_grid(d, n, _p(sorted_pts), _p(sorted_keys), _p(grid_ds),
                                                          _p(grid_size), _p(radii), _p(selected), ctypes.byref(count),
                                                          ws.data_ptr(), ws.numel(), _stream()),
                    "poisson_disk_sampling_grid")
    return selected[:count.value].reshape(-1, 1)


# ---- dense contraction -----------------------------------------------------------------------
def gemm_f32(a, b, split=True):
    """a [M, K] @ b[N, K]^T -> [M, N] float32 on the tcgen05 tensor cores (bf16 hi/lo split when
    `split`, one bf16 pass otherwise).  Stand-in for the torch::matmul calls of the reference's
    pcconvs/kpconv.cu:56-57 and mcconv.cu:64-68."""
    a = _need(a, "a", torch.float32, 2)
    b = _need(b, "b", torch.float32, 2)
    if a.shape[1] != b.shape[1]:
        raise RuntimeError("gemm_f32: inner dimensions differ")
    m, k = a.shape
    n = b.shape[0]
    out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    if n == 0 or k == 0:
        return out.zero_()
    with _on(a.device):
        ws = _workspace(_lib.pccnn_gemm_workspace_bytes(m, n, k), a.device)
        _capi.check(_lib.pccnn_gemm_f32(m, n, k, _p(a), a.stride(0), _p(b), b.stride(0), _p(out), out.stride(0),
                                        1 if split else 0, ws.data_ptr(), ws.numel(), _stream()), "gemm_f32")
    return out


# ---- point convolutions ----------------------------------------------------------------------
def _conv_common(pts, feats, samples, neighbors, start_ids, radii, feat_dtype=torch.float32):
    pts = _need(pts, "pts", torch.float32, 2)
    feats = _need(feats, "features", feat_dtype, 2)
    samples = _need(samples, "samples", torch.float32, 2)
    neighbors = _need(neighbors, "neighbors", torch.int32, 2)
    start_ids = _need(start_ids, "start_ids", torch.int32, 1)
    radii = _need(radii, "radii", torch.float32, 1)
    d = _dims(pts)
    if samples.shape[1] != d or radii.numel() != d:
        raise RuntimeError("samples and radii must match the point dimension %d" % d)
    if feats.shape[0] != pts.shape[0]:
        raise RuntimeError("features need one row per point")
    if start_ids.shape[0] != samples.shape[0]:
        raise RuntimeError("start_ids needs one entry per sample")
    if neighbors.shape[1] != 2:
        raise RuntimeError("neighbors must be [T, 2]")
    _maybe_validate(neighbors, start_ids, pts.shape[0])
    return pts, feats, samples, neighbors, start_ids, radii, d


def kp_conv(pts, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights):
    """KPConv forward -> [M, Cout]; kpconv() of pccnn_lib_ops/pcconvs/kpconv.cu:32-60 of the reference.
    bfloat16 features with bfloat16 weights select the single-pass inference path (bfloat16 output)."""
    if isinstance(feats, torch.Tensor) and feats.dtype == torch.bfloat16:
        return _kp_conv_bf16(pts, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights)
    pts, feats, samples, neighbors, start_ids, radii, d = _conv_common(pts, feats, samples, neighbors, start_ids, radii)
    kernel_pts = _need(kernel_pts, "kernel_pts", torch.float32, 2)
    weights = _need(weights, "weights", torch.float32, 2)
    k, cin, cout = kernel_pts.shape[0], feats.shape[1], weights.shape[1]
    if kernel_pts.shape[1] != d or weights.shape[0] != k * cin:
        raise RuntimeError("kernel_pts must be [K, %d] and weights [K * Cin, Cout]" % d)
    m = samples.shape[0]
    out = torch.empty((m, cout), dtype=torch.float32, device=pts.device)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_conv_workspace_bytes(feats.shape[0], m, cin, k, cout), pts.device)
        _capi.check(_lib.pccnn_kp_conv(d, pts.shape[0], _p(pts), _p(feats), cin, m, _p(samples), _p(neighbors),
                                       _p(start_ids), _p(radii), _p(kernel_pts), k, float(sigma), _p(weights), cout,
                                       _p(out), ws.data_ptr(), ws.numel(), _stream()), "kp_conv")
    return out


def kp_conv_grid(sorted_pts, sorted_keys, sorted_ids, feats, samples, sample_keys, grid_ds, grid_size, radii, kernel_pts,
                 sigma, weights):
    """KPConv forward without a neighbor list -> [M, Cout]: the kernel searches the grid itself (3-D points, radius =
    cell size).  `sorted_pts` / `sorted_keys` / `sorted_ids` / `grid_ds` / `grid_size` as a Grid holds them, `feats` in
    the original point order, `samples` with their keys on the same grid.  Same result as find_neighbors + kp_conv;
    float32 or bfloat16 features (with weights of the same dtype).  No counterpart in the reference, where every
    convolution reads a materialised list (pccnn_lib/pc/layers/KPConv.py:127-146)."""
    sorted_pts = _need(sorted_pts, "sorted_pts", torch.float32, 2)
    sorted_keys = _need(sorted_keys, "sorted_keys", torch.int64, 1)
    if sorted_ids is not None:
        sorted_ids = _need(sorted_ids, "sorted_ids", torch.int64, 1)
    samples = _need(samples, "samples", torch.float32, 2)
    sample_keys = _need(sample_keys, "sample_keys", torch.int64, 1)
    grid_ds = _need(grid_ds, "grid_ds", torch.int32)
    grid_size = _need(grid_size, "grid_size", torch.int32, 1)
    radii = _need(radii, "radii", torch.float32, 1)
    kernel_pts = _need(kernel_pts, "kernel_pts", torch.float32, 2)
    bf16 = isinstance(feats, torch.Tensor) and feats.dtype == torch.bfloat16
    feats = _need(feats, "features", torch.bfloat16 if bf16 else torch.float32, 2)
    weights = _need(weights, "weights", torch.bfloat16 if bf16 else torch.float32, 2)
    if sorted_pts.shape[1] != 3 or samples.shape[1] != 3 or kernel_pts.shape[1] != 3:
        raise RuntimeError("kp_conv_grid is defined for 3-D points")
    n, m, cin, k, cout = sorted_pts.shape[0], samples.shape[0], feats.shape[1], kernel_pts.shape[0], weights.shape[1]
    if feats.shape[0] != n or sorted_keys.shape[0] != n or sample_keys.shape[0] != m or weights.shape[0] != k * cin:
        raise RuntimeError("kp_conv_grid: sizes of points / keys / features / weights do not match")
    out = torch.empty((m, cout), dtype=feats.dtype, device=feats.device)
    with _on(feats.device):
        ws = _workspace(_lib.pccnn_kp_conv_grid_workspace_bytes(n, m, cin, k, cout), feats.device)
        _capi.check(_lib.pccnn_kp_conv_grid(n, _p(sorted_pts), _p(sorted_keys), _p(sorted_ids), _p(feats), 1 if bf16 else 0,
                                            cin, m, _p(samples), _p(sample_keys), _p(grid_ds), _p(grid_size), _p(radii),
                                            _p(kernel_pts), k, float(sigma), _p(weights), cout, _p(out), ws.data_ptr(),
                                            ws.numel(), _stream()), "kp_conv_grid")
    return out


def _kp_conv_bf16(pts, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights):
    pts, feats, samples, neighbors, start_ids, radii, d = _conv_common(pts, feats, samples, neighbors, start_ids, radii,
                                                                        torch.bfloat16)
    kernel_pts = _need(kernel_pts, "kernel_pts", torch.float32, 2)
    weights = _need(weights, "weights", torch.bfloat16, 2)
    k, cin, cout = kernel_pts.shape[0], feats.shape[1], weights.shape[1]
    if d != 3 or kernel_pts.shape[1] != d or weights.shape[0] != k * cin:
        raise RuntimeError("bfloat16 KPConv needs 3-D points, kernel_pts [K, 3] and weights [K * Cin, Cout]")
    m = samples.shape[0]
    out = torch.empty((m, cout), dtype=torch.bfloat16, device=pts.device)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_conv_workspace_bytes(feats.shape[0], m, cin, k, cout), pts.device)
        _capi.check(_lib.pccnn_kp_conv_bf16(d, pts.shape[0], _p(pts), _p(feats), cin, m, _p(samples), _p(neighbors),
                                            _p(start_ids), _p(radii), _p(kernel_pts), k, float(sigma), _p(weights),
                                            cout, _p(out), ws.data_ptr(), ws.numel(), _stream()), "kp_conv_bf16")
    return out


def mc_conv(pts, pdf, feats, samples, neighbors, start_ids, radii, axis_proj, axis_bias, weights):
    """MCConv forward -> [M, Cout]; mcconv() of pccnn_lib_ops/pcconvs/mcconv.cu:32-71 of the reference."""
    pts, feats, samples, neighbors, start_ids, radii, d = _conv_common(pts, feats, samples, neighbors, start_ids, radii)
    pdf = _need(pdf, "pdf", torch.float32, 1)
    axis_proj = _need(axis_proj, "axis_proj", torch.float32, 2)
    axis_bias = _need(axis_bias, "axis_bias", torch.float32)
    weights = _need(weights, "weights", torch.float32, 3)
    hidden, cin = axis_proj.shape[1], feats.shape[1]
    n_mlps = weights.shape[0]
    cout = weights.shape[2] * n_mlps
    if axis_proj.shape[0] != d or axis_bias.numel() != hidden or weights.shape[1] * n_mlps != hidden * cin:
        raise RuntimeError("axis_proj must be [%d, H], axis_bias [1, H] and weights [mlps, H * Cin / mlps, Cout / mlps]" % d)
    m = samples.shape[0]
    out = torch.empty((m, cout), dtype=torch.float32, device=pts.device)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_conv_workspace_bytes(feats.shape[0], m, cin, hidden, cout), pts.device)
        _capi.check(_lib.pccnn_mc_conv(d, pts.shape[0], _p(pts), _p(pdf), _p(feats), cin, m, _p(samples), _p(neighbors),
                                       _p(start_ids), _p(radii), _p(axis_proj), _p(axis_bias), hidden, n_mlps,
                                       _p(weights), cout, _p(out), ws.data_ptr(), ws.numel(), _stream()), "mc_conv")
    return out


def gemm_bf16(a_hi, b_hi, a_lo=None, b_lo=None, out=None, status=None):
    """The tensor-core kernel alone on bf16 operands a [M, K], b [N, K] (K a multiple of 64, optional
    low parts for the three-product split) -> [M, N] float32.  Asynchronous; `status` (int32 tensor
    of one element) is set non-zero by the kernel if one of its bounded waits ran out."""
    a_hi = _need(a_hi, "a_hi", torch.bfloat16, 2)
    b_hi = _need(b_hi, "b_hi", torch.bfloat16, 2)
    if (a_lo is None) != (b_lo is None):
        raise RuntimeError("gemm_bf16: give the low parts of both operands or of neither")
    if a_lo is not None:
        a_lo = _need(a_lo, "a_lo", torch.bfloat16, 2)
        b_lo = _need(b_lo, "b_lo", torch.bfloat16, 2)
    m, k = a_hi.shape
    n = b_hi.shape[0]
    if k % 64 or b_hi.shape[1] != k:
        raise RuntimeError("gemm_bf16: K must match and be a multiple of 64")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a_hi.device)
    if status is None:
        status = torch.zeros((1,), dtype=torch.int32, device=a_hi.device)
    with _on(a_hi.device):
        _capi.check(_lib.pccnn_gemm_bf16(m, n, k, _p(a_hi), _p(a_lo), a_hi.stride(0), _p(b_hi), _p(b_lo), b_hi.stride(0),
                                         _p(out), out.stride(0), _p(status), _stream()), "gemm_bf16")
    return out


def gemm_tn_f32(a, b, split=True):
    """a[R, I]^T @ b[R, N] -> [I, N] float32 on the tensor cores (reduction over the rows): the
    weight-gradient contraction of pcconvs/kpconv.cu:90-93 of the reference."""
    a = _need(a, "a", torch.float32, 2)
    b = _need(b, "b", torch.float32, 2)
    if a.shape[0] != b.shape[0]:
        raise RuntimeError("gemm_tn_f32: row counts differ")
    r, i = a.shape
    n = b.shape[1]
    out = torch.zeros((i, n), dtype=torch.float32, device=a.device)
    if r == 0 or i == 0 or n == 0:
        return out
    with _on(a.device):
        ws = _workspace(_lib.pccnn_gemm_tn_workspace_bytes(r, i, n), a.device)
        _capi.check(_lib.pccnn_gemm_tn_f32(r, i, n, _p(a), a.stride(0), _p(b), b.stride(0), _p(out), out.stride(0),
                                           1 if split else 0, ws.data_ptr(), ws.numel(), _stream()), "gemm_tn_f32")
    return out


def _arm_weight_grads_event(event):
    if event is not None:
        if not event.cuda_event:
            event.record()  # torch creates the underlying CUDA event at its first record
        _capi.check(_lib.pccnn_conv_grads_set_weight_grads_event(event.cuda_event), "set_weight_grads_event")


def kp_conv_grads(pts, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights, in_grads,
                  weight_grads_event=None):
    """[dW, dFeat, dKernelPts, dPts, dSamples]; kpconv_grads() of pccnn_lib_ops/pcconvs/kpconv.cu:63-112.
    `weight_grads_event` (an extension for data parallelism): a torch.cuda.Event that is recorded on the current
    stream as soon as dW is final, before the rest of the backward pass has run."""
    pts, feats, samples, neighbors, start_ids, radii, d = _conv_common(pts, feats, samples, neighbors, start_ids, radii)
    kernel_pts = _need(kernel_pts, "kernel_pts", torch.float32, 2)
    weights = _need(weights, "weights", torch.float32, 2)
    in_grads = _need(in_grads, "in_grads", torch.float32, 2)
    k, cin, cout = kernel_pts.shape[0], feats.shape[1], weights.shape[1]
    m, n = samples.shape[0], pts.shape[0]
    if weights.shape[0] != k * cin or tuple(in_grads.shape) != (m, cout):
        raise RuntimeError("weights must be [K * Cin, Cout] and in_grads [M, Cout]")
    dev = pts.device
    d_w, d_f = torch.empty_like(weights), torch.empty_like(feats)
    d_k, d_p, d_s = torch.empty_like(kernel_pts), torch.empty_like(pts), torch.empty_like(samples)
    with _on(dev):
        ws = _workspace(_lib.pccnn_conv_grads_workspace_bytes(feats.shape[0], m, cin, k, cout), dev)
        _arm_weight_grads_event(weight_grads_event)
        _capi.check(_lib.pccnn_kp_conv_grads(d, n, _p(pts), _p(feats), cin, m, _p(samples), _p(neighbors),
                                             _p(start_ids), _p(radii), _p(kernel_pts), k, float(sigma), _p(weights),
                                             cout, _p(in_grads), d_w.data_ptr(), d_f.data_ptr(), d_k.data_ptr(),
                                             d_p.data_ptr(), d_s.data_ptr(), ws.data_ptr(), ws.numel(), _stream()),
                    "kp_conv_grads")
    return [d_w, d_f, d_k, d_p, d_s]


def mc_conv_grads(pts, pdf, feats, samples, neighbors, start_ids, radii, axis_proj, axis_bias, weights, in_grads,
                  weight_grads_event=None):
    """[dW, dFeat, dAxis, dBias, dPdf, dPts, dSamples]; mcconv_grads() of pccnn_lib_ops/pcconvs/mcconv.cu:73-143.
    `weight_grads_event`: as for kp_conv_grads."""
    pts, feats, samples, neighbors, start_ids, radii, d = _conv_common(pts, feats, samples, neighbors, start_ids, radii)
    pdf = _need(pdf, "pdf", torch.float32, 1)
    axis_proj = _need(axis_proj, "axis_proj", torch.float32, 2)
    axis_bias = _need(axis_bias, "axis_bias", torch.float32)
    weights = _need(weights, "weights", torch.float32, 3)
    in_grads = _need(in_grads, "in_grads", torch.float32, 2)
    hidden, cin, n_mlps = axis_proj.shape[1], feats.shape[1], weights.shape[0]
    cout = weights.shape[2] * n_mlps
    m, n = samples.shape[0], pts.shape[0]
    if tuple(in_grads.shape) != (m, cout):
        raise RuntimeError("in_grads must be [M, Cout]")
    dev = pts.device
    d_w, d_f = torch.empty_like(weights), torch.empty_like(feats)
    d_a, d_b, d_pdf = torch.empty_like(axis_proj), torch.empty_like(axis_bias), torch.empty_like(pdf)
    d_p, d_s = torch.empty_like(pts), torch.empty_like(samples)
    with _on(dev):
        ws = _workspace(_lib.pccnn_conv_grads_workspace_bytes(feats.shape[0], m, cin, hidden, cout), dev)
        _arm_weight_grads_event(weight_grads_event)
        _capi.check(_lib.pccnn_mc_conv_grads(d, n, _p(pts), _p(pdf), _p(feats), cin, m, _p(samples), _p(neighbors),
                                             _p(start_ids), _p(radii), _p(axis_proj), _p(axis_bias), hidden, n_mlps,
                                             _p(weights), cout, _p(in_grads), d_w.data_ptr(), d_f.data_ptr(),
                                             d_a.data_ptr(), d_b.data_ptr(), d_pdf.data_ptr(), d_p.data_ptr(),
                                             d_s.data_ptr(), ws.data_ptr(), ws.numel(), _stream()), "mc_conv_grads")
    return [d_w, d_f, d_a, d_b, d_pdf, d_p, d_s]


# ---- weight variance (variance-aware initialisation) ---------------------------------------------
def _variance_out(device):
    return torch.empty((), dtype=torch.float32, device=device)


def kp_conv_weight_var(pts, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma):
    """0-dim tensor 1 / mean_m ||P[m]||^2; kpconv_compute_weight_variance() of pccnn_lib_ops/pcconvs/kpconv.cu:115-135."""
    pts, feats, samples, neighbors, start_ids, radii, d = _conv_common(pts, feats, samples, neighbors, start_ids, radii)
    kernel_pts = _need(kernel_pts, "kernel_pts", torch.float32, 2)
    k, cin, m = kernel_pts.shape[0], feats.shape[1], samples.shape[0]
    out = _variance_out(pts.device)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_conv_weight_var_workspace_bytes(feats.shape[0], m, cin, k), pts.device)
        _capi.check(_lib.pccnn_kp_conv_weight_var(d, pts.shape[0], _p(pts), _p(feats), cin, m, _p(samples), _p(neighbors),
                                                  _p(start_ids), _p(radii), _p(kernel_pts), k, float(sigma), out.data_ptr(),
                                                  ws.data_ptr(), ws.numel(), _stream()), "kp_conv_weight_var")
    return out


def mc_conv_weight_var(pts, pdf, feats, samples, neighbors, start_ids, radii, axis_proj, axis_bias):
    """mcconv_compute_weight_variance() of pccnn_lib_ops/pcconvs/mcconv.cu:146-171."""
    pts, feats, samples, neighbors, start_ids, radii, d = _conv_common(pts, feats, samples, neighbors, start_ids, radii)
    pdf = _need(pdf, "pdf", torch.float32, 1)
    axis_proj = _need(axis_proj, "axis_proj", torch.float32, 2)
    axis_bias = _need(axis_bias, "axis_bias", torch.float32)
    hidden, cin, m = axis_proj.shape[1], feats.shape[1], samples.shape[0]
    out = _variance_out(pts.device)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_conv_weight_var_workspace_bytes(feats.shape[0], m, cin, hidden), pts.device)
        _capi.check(_lib.pccnn_mc_conv_weight_var(d, pts.shape[0], _p(pts), _p(pdf), _p(feats), cin, m, _p(samples),
                                                  _p(neighbors), _p(start_ids), _p(radii), _p(axis_proj), _p(axis_bias),
                                                  hidden, out.data_ptr(), ws.data_ptr(), ws.numel(), _stream()),
                    "mc_conv_weight_var")
    return out


# ---- KPConvN and PCCNN -------------------------------------------------------------------------------
def _kp_density_args(pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, weights=None, in_grads=None):
    pts, feats, samples, neighbors, start_ids, radii, d = _conv_common(pts, feats, samples, neighbors, start_ids, radii)
    pdf = _need(pdf, "pdf", torch.float32, 1)
    kernel_pts = _need(kernel_pts, "kernel_pts", torch.float32, 2)
    k, cin = kernel_pts.shape[0], feats.shape[1]
    if kernel_pts.shape[1] != d or pdf.shape[0] != pts.shape[0]:
        raise RuntimeError("kernel_pts must be [K, %d] and pdf must have one entry per point" % d)
    cout = None
    if weights is not None:
        weights = _need(weights, "weights", torch.float32, 2)
        if weights.shape[0] != k * cin:
            raise RuntimeError("weights must be [K * Cin, Cout]")
        cout = weights.shape[1]
    if in_grads is not None:
        in_grads = _need(in_grads, "in_grads", torch.float32, 2)
        if tuple(in_grads.shape) != (samples.shape[0], cout):
            raise RuntimeError("in_grads must be [M, Cout]")
    return pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, weights, in_grads, d, k, cin, cout


def kp_conv_n(pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights):
    """KPConvN forward (kernel-point basis divided by the neighbor's density); kpconvn() of
    pccnn_lib_ops/pcconvs/kpconvn.cu:32-68."""
    pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, weights, _, d, k, cin, cout = _kp_density_args(
        pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, weights)
    m = samples.shape[0]
    out = torch.empty((m, cout), dtype=torch.float32, device=pts.device)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_conv_workspace_bytes(feats.shape[0], m, cin, k, cout), pts.device)
        _capi.check(_lib.pccnn_kp_conv_n(d, pts.shape[0], _p(pts), _p(pdf), _p(feats), cin, m, _p(samples), _p(neighbors),
                                         _p(start_ids), _p(radii), _p(kernel_pts), k, float(sigma), _p(weights), cout,
                                         _p(out), ws.data_ptr(), ws.numel(), _stream()), "kp_conv_n")
    return out


def kp_conv_n_grads(pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights, in_grads):
    """[dW, dFeat, dKernelPts, dPts, dSamples]; kpconvn_grads() of pccnn_lib_ops/pcconvs/kpconvn.cu:71-130."""
    pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, weights, in_grads, d, k, cin, cout = \
        _kp_density_args(pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, weights, in_grads)
    m, n, dev = samples.shape[0], pts.shape[0], pts.device
    d_w, d_f = torch.empty_like(weights), torch.empty_like(feats)
    d_k, d_p, d_s = torch.empty_like(kernel_pts), torch.empty_like(pts), torch.empty_like(samples)
    with _on(dev):
        ws = _workspace(_lib.pccnn_conv_grads_workspace_bytes(feats.shape[0], m, cin, k, cout), dev)
        _capi.check(_lib.pccnn_kp_conv_n_grads(d, n, _p(pts), _p(pdf), _p(feats), cin, m, _p(samples), _p(neighbors),
                                               _p(start_ids), _p(radii), _p(kernel_pts), k, float(sigma), _p(weights), cout,
                                               _p(in_grads), d_w.data_ptr(), d_f.data_ptr(), d_k.data_ptr(), d_p.data_ptr(),
                                               d_s.data_ptr(), ws.data_ptr(), ws.numel(), _stream()), "kp_conv_n_grads")
    return [d_w, d_f, d_k, d_p, d_s]


def kp_conv_n_weight_var(pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, sigma):
    """kpconvn_compute_weight_variance() of pccnn_lib_ops/pcconvs/kpconvn.cu:133-155."""
    pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, _, _, d, k, cin, _ = _kp_density_args(
        pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts)
    m = samples.shape[0]
    out = _variance_out(pts.device)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_conv_weight_var_workspace_bytes(feats.shape[0], m, cin, k), pts.device)
        _capi.check(_lib.pccnn_kp_conv_n_weight_var(d, pts.shape[0], _p(pts), _p(pdf), _p(feats), cin, m, _p(samples),
                                                    _p(neighbors), _p(start_ids), _p(radii), _p(kernel_pts), k, float(sigma),
                                                    out.data_ptr(), ws.data_ptr(), ws.numel(), _stream()),
                    "kp_conv_n_weight_var")
    return out


def pccnn(pts, feats, pdf, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights):
    """PCCNN forward (Gaussian kernel-point basis divided by the density); pccnn() of pccnn_lib_ops/pcconvs/pccnn.cu:32-66.
    Argument order as there: features before the density."""
    pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, weights, _, d, k, cin, cout = _kp_density_args(
        pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, weights)
    m = samples.shape[0]
    out = torch.empty((m, cout), dtype=torch.float32, device=pts.device)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_conv_workspace_bytes(feats.shape[0], m, cin, k, cout), pts.device)
        _capi.check(_lib.pccnn_pccnn_conv(d, pts.shape[0], _p(pts), _p(feats), cin, _p(pdf), m, _p(samples), _p(neighbors),
                                          _p(start_ids), _p(radii), _p(kernel_pts), k, float(sigma), _p(weights), cout,
                                          _p(out), ws.data_ptr(), ws.numel(), _stream()), "pccnn")
    return out


def pccnn_grads(pts, feats, pdf, samples, neighbors, start_ids, radii, kernel_pts, sigma, weights, in_grads):
    """[dW, dFeat, dKernelPts, dPdf, dPts, dSamples]; pccnn_grads() of pccnn_lib_ops/pcconvs/pccnn.cu:69-139."""
    pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, weights, in_grads, d, k, cin, cout = \
        _kp_density_args(pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, weights, in_grads)
    m, n, dev = samples.shape[0], pts.shape[0], pts.device
    d_w, d_f, d_k = torch.empty_like(weights), torch.empty_like(feats), torch.empty_like(kernel_pts)
    d_pdf, d_p, d_s = torch.empty_like(pdf), torch.empty_like(pts), torch.empty_like(samples)
    with _on(dev):
        ws = _workspace(_lib.pccnn_conv_grads_workspace_bytes(feats.shape[0], m, cin, k, cout), dev)
        _capi.check(_lib.pccnn_pccnn_conv_grads(d, n, _p(pts), _p(feats), cin, _p(pdf), m, _p(samples), _p(neighbors),
                                                _p(start_ids), _p(radii), _p(kernel_pts), k, float(sigma), _p(weights), cout,
                                                _p(in_grads), d_w.data_ptr(), d_f.data_ptr(), d_k.data_ptr(),
                                                d_pdf.data_ptr(), d_p.data_ptr(), d_s.data_ptr(), ws.data_ptr(), ws.numel(),
                                                _stream()), "pccnn_grads")
    return [d_w, d_f, d_k, d_pdf, d_p, d_s]


def pccnn_weight_variance(pts, feats, pdf, samples, neighbors, start_ids, radii, kernel_pts, sigma):
    """pccnn_compute_weight_variance() of pccnn_lib_ops/pcconvs/pccnn.cu:142-165."""
    pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts, _, _, d, k, cin, _ = _kp_density_args(
        pts, pdf, feats, samples, neighbors, start_ids, radii, kernel_pts)
    m = samples.shape[0]
    out = _variance_out(pts.device)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_conv_weight_var_workspace_bytes(feats.shape[0], m, cin, k), pts.device)
        _capi.check(_lib.pccnn_pccnn_conv_weight_var(d, pts.shape[0], _p(pts), _p(feats), cin, _p(pdf), m, _p(samples),
                                                     _p(neighbors), _p(start_ids), _p(radii), _p(kernel_pts), k,
                                                     float(sigma), out.data_ptr(), ws.data_ptr(), ws.numel(), _stream()),
                    "pccnn_weight_variance")
    return out


# ---- SPHConv -----------------------------------------------------------------------------------------
def _sph_args(pts, feats, samples, neighbors, start_ids, radii, radial_bins, azimuz_bins, polar_bins):
    pts, feats, samples, neighbors, start_ids, radii, d = _conv_common(pts, feats, samples, neighbors, start_ids, radii)
    if d != 3:
        raise RuntimeError("SPHConv is defined for 3-D points only")
    bins = [_need(b, n, torch.float32, 1) for b, n in ((radial_bins, "radial_bins"), (azimuz_bins, "azimuz_bins"),
                                                        (polar_bins, "polar_bins"))]
    k = bins[0].numel() * bins[1].numel() * bins[2].numel() + 1
    return pts, feats, samples, neighbors, start_ids, radii, bins, k


def _bins_c(bins):
    return (_p(bins[0]), bins[0].numel(), _p(bins[1]), bins[1].numel(), _p(bins[2]), bins[2].numel())


def sph_conv(pts, feats, samples, neighbors, start_ids, radii, radial_bins, azimuz_bins, polar_bins, weights):
    """SPHConv forward -> [M, Cout]; sphconv() of pccnn_lib_ops/pcconvs/sphconv.cu:32-72."""
    pts, feats, samples, neighbors, start_ids, radii, bins, k = _sph_args(pts, feats, samples, neighbors, start_ids, radii,
                                                                           radial_bins, azimuz_bins, polar_bins)
    weights = _need(weights, "weights", torch.float32, 2)
    cin, cout, m = feats.shape[1], weights.shape[1], samples.shape[0]
    if weights.shape[0] != k * cin:
        raise RuntimeError("weights must be [(R * A * P + 1) * Cin, Cout]")
    out = torch.empty((m, cout), dtype=torch.float32, device=pts.device)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_conv_workspace_bytes(feats.shape[0], m, cin, k, cout), pts.device)
        _capi.check(_lib.pccnn_sph_conv(3, pts.shape[0], _p(pts), _p(feats), cin, m, _p(samples), _p(neighbors), _p(start_ids),
                                        _p(radii), *_bins_c(bins), _p(weights), cout, _p(out), ws.data_ptr(), ws.numel(),
                                        _stream()), "sph_conv")
    return out


def sph_conv_grads(pts, feats, samples, neighbors, start_ids, radii, radial_bins, azimuz_bins, polar_bins, weights,
                   in_grads):
    """[dW, dFeat]; sphconv_grads() of pccnn_lib_ops/pcconvs/sphconv.cu:75-120."""
    pts, feats, samples, neighbors, start_ids, radii, bins, k = _sph_args(pts, feats, samples, neighbors, start_ids, radii,
                                                                           radial_bins, azimuz_bins, polar_bins)
    weights = _need(weights, "weights", torch.float32, 2)
    in_grads = _need(in_grads, "in_grads", torch.float32, 2)
    cin, cout, m = feats.shape[1], weights.shape[1], samples.shape[0]
    if weights.shape[0] != k * cin or tuple(in_grads.shape) != (m, cout):
        raise RuntimeError("weights must be [(R * A * P + 1) * Cin, Cout] and in_grads [M, Cout]")
    d_w, d_f = torch.empty_like(weights), torch.empty_like(feats)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_conv_grads_workspace_bytes(feats.shape[0], m, cin, k, cout), pts.device)
        _capi.check(_lib.pccnn_sph_conv_grads(3, pts.shape[0], _p(pts), _p(feats), cin, m, _p(samples), _p(neighbors),
                                              _p(start_ids), _p(radii), *_bins_c(bins), _p(weights), cout, _p(in_grads),
                                              d_w.data_ptr(), d_f.data_ptr(), ws.data_ptr(), ws.numel(), _stream()),
                    "sph_conv_grads")
    return [d_w, d_f]


def sph_conv_weight_var(pts, feats, samples, neighbors, start_ids, radii, radial_bins, azimuz_bins, polar_bins):
    """sphconv_compute_weight_variance() of pccnn_lib_ops/pcconvs/sphconv.cu:123-146."""
    pts, feats, samples, neighbors, start_ids, radii, bins, k = _sph_args(pts, feats, samples, neighbors, start_ids, radii,
                                                                           radial_bins, azimuz_bins, polar_bins)
    cin, m = feats.shape[1], samples.shape[0]
    out = _variance_out(pts.device)
    with _on(pts.device):
        ws = _workspace(_lib.pccnn_conv_weight_var_workspace_bytes(feats.shape[0], m, cin, k), pts.device)
        _capi.check(_lib.pccnn_sph_conv_weight_var(3, pts.shape[0], _p(pts), _p(feats), cin, m, _p(samples), _p(neighbors),
                                                   _p(start_ids), _p(radii), *_bins_c(bins), out.data_ptr(), ws.data_ptr(),
                                                   ws.numel(), _stream()), "sph_conv_weight_var")
    return out


# ---- PointConv ---------------------------------------------------------------------------------------
def point_conv_basis(pts, radii, samples, neighbors, axis_proj, axis_bias):
    """[T, H] affine projection of the normalised offsets; pointconv_basis() of pccnn_lib_ops/pcconvs/pointconv.cu:32-51."""
    pts = _need(pts, "pts", torch.float32, 2)
    radii = _need(radii, "radii", torch.float32, 1)
    samples = _need(samples, "samples", torch.float32, 2)
    neighbors = _need(neighbors, "neighbors", torch.int32, 2)
    axis_proj = _need(axis_proj, "axis_proj", torch.float32, 2)
    axis_bias = _need(axis_bias, "axis_bias", torch.float32)
    d, hidden, t = _dims(pts), axis_proj.shape[1], neighbors.shape[0]
    if samples.shape[1] != d or radii.numel() != d or axis_proj.shape[0] != d or axis_bias.numel() != hidden:
        raise RuntimeError("samples, radii, axis_proj [D, H] and axis_bias [1, H] must match the point dimension %d" % d)
    out = torch.empty((t, hidden), dtype=torch.float32, device=pts.device)
    with _on(pts.device):
        _capi.check(_lib.pccnn_point_conv_basis(d, t, _p(pts), _p(radii), _p(samples), _p(neighbors), _p(axis_proj),
                                                _p(axis_bias), hidden, _p(out), _stream()), "point_conv_basis")
    return out


def point_conv_basis_grads(pts, radii, samples, neighbors, axis_proj, axis_bias, in_grads):
    """[dPts, dSamples, dAxis, dBias]; pointconv_basis_grads() of pccnn_lib_ops/pcconvs/pointconv.cu:54-86."""
    pts = _need(pts, "pts", torch.float32, 2)
    radii = _need(radii, "radii", torch.float32, 1)
    samples = _need(samples, "samples", torch.float32, 2)
    neighbors = _need(neighbors, "neighbors", torch.int32, 2)
    axis_proj = _need(axis_proj, "axis_proj", torch.float32, 2)
    axis_bias = _need(axis_bias, "axis_bias", torch.float32)
    in_grads = _need(in_grads, "in_grads", torch.float32, 2)
    d, hidden, t = _dims(pts), axis_proj.shape[1], neighbors.shape[0]
    if tuple(in_grads.shape) != (t, hidden):
        raise RuntimeError("in_grads must be [T, H]")
    d_p, d_s = torch.empty_like(pts), torch.empty_like(samples)
    d_a, d_b = torch.empty_like(axis_proj), torch.empty((1, hidden), dtype=torch.float32, device=pts.device)
    with _on(pts.device):
        _capi.check(_lib.pccnn_point_conv_basis_grads(d, pts.shape[0], samples.shape[0], t, _p(pts), _p(radii), _p(samples),
                                                      _p(neighbors), _p(axis_proj), hidden, _p(in_grads), d_p.data_ptr(),
                                                      d_s.data_ptr(), d_a.data_ptr(), d_b.data_ptr(), _stream()),
                    "point_conv_basis_grads")
    return [d_p, d_s, d_a, d_b]


def _point_conv_args(basis, feats, neighbors, start_ids):
    basis = _need(basis, "basis", torch.float32, 2)
    feats = _need(feats, "features", torch.float32, 2)
    neighbors = _need(neighbors, "neighbors", torch.int32, 2)
    start_ids = _need(start_ids, "start_ids", torch.int32, 1)
    if basis.shape[0] != neighbors.shape[0] or neighbors.shape[1] != 2:
        raise RuntimeError("basis needs one row per neighbor pair")
    if basis.shape[1] > 64:
        raise RuntimeError("at most 64 basis functions are supported (got %d)" % basis.shape[1])
    _maybe_validate(neighbors, start_ids, feats.shape[0])
    return basis, feats, neighbors, start_ids


def point_conv(basis, feats, neighbors, start_ids, weights):
    """PointConv contraction on a caller-made basis [T, H] -> [M, Cout]; pointconv() of pointconv.cu:89-103."""
    basis, feats, neighbors, start_ids = _point_conv_args(basis, feats, neighbors, start_ids)
    weights = _need(weights, "weights", torch.float32, 2)
    hidden, cin, cout, m = basis.shape[1], feats.shape[1], weights.shape[1], start_ids.shape[0]
    if weights.shape[0] != hidden * cin:
        raise RuntimeError("weights must be [H * Cin, Cout]")
    out = torch.empty((m, cout), dtype=torch.float32, device=feats.device)
    with _on(feats.device):
        ws = _workspace(_lib.pccnn_conv_workspace_bytes(feats.shape[0], m, cin, hidden, cout), feats.device)
        _capi.check(_lib.pccnn_point_conv(feats.shape[0], _p(basis), hidden, _p(feats), cin, m, _p(neighbors), _p(start_ids),
                                          _p(weights), cout, _p(out), ws.data_ptr(), ws.numel(), _stream()), "point_conv")
    return out


def point_conv_grads(basis, feats, neighbors, start_ids, weights, in_grads):
    """[dW, dFeat, dBasis]; pointconv_grads() of pccnn_lib_ops/pcconvs/pointconv.cu:106-127."""
    basis, feats, neighbors, start_ids = _point_conv_args(basis, feats, neighbors, start_ids)
    weights = _need(weights, "weights", torch.float32, 2)
    in_grads = _need(in_grads, "in_grads", torch.float32, 2)
    hidden, cin, cout, m = basis.shape[1], feats.shape[1], weights.shape[1], start_ids.shape[0]
    if weights.shape[0] != hidden * cin or tuple(in_grads.shape) != (m, cout):
        raise RuntimeError("weights must be [H * Cin, Cout] and in_grads [M, Cout]")
    d_w, d_f, d_b = torch.empty_like(weights), torch.empty_like(feats), torch.empty_like(basis)
    with _on(feats.device):
        ws = _workspace(_lib.pccnn_conv_grads_workspace_bytes(feats.shape[0], m, cin, hidden, cout), feats.device)
        _capi.check(_lib.pccnn_point_conv_grads(feats.shape[0], _p(basis), hidden, _p(feats), cin, m, basis.shape[0],
                                                _p(neighbors), _p(start_ids), _p(weights), cout, _p(in_grads),
                                                d_w.data_ptr(), d_f.data_ptr(), d_b.data_ptr(), ws.data_ptr(), ws.numel(),
                                                _stream()), "point_conv_grads")
    return [d_w, d_f, d_b]


def point_conv_weight_var(basis, feats, neighbors, start_ids):
    """pointconv_compute_weight_variance() of pccnn_lib_ops/pcconvs/pointconv.cu:130-139."""
    basis, feats, neighbors, start_ids = _point_conv_args(basis, feats, neighbors, start_ids)
    hidden, cin, m = basis.shape[1], feats.shape[1], start_ids.shape[0]
    out = _variance_out(feats.device)
    with _on(feats.device):
        ws = _workspace(_lib.pccnn_conv_weight_var_workspace_bytes(feats.shape[0], m, cin, hidden), feats.device)
        _capi.check(_lib.pccnn_point_conv_weight_var(feats.shape[0], _p(basis), hidden, _p(feats), cin, m, _p(neighbors),
                                                     _p(start_ids), out.data_ptr(), ws.data_ptr(), ws.numel(), _stream()),
                    "point_conv_weight_var")
    return out
