"""ctypes binding of libpccnn_b200.so (declared in include/pccnn_b200.h).

There is no fallback: if the library cannot be loaded the import raises, and every compute
call raises ``RuntimeError`` when the C entry point reports an error.
"""
import ctypes
import os

from . import _build

_c_i64 = ctypes.c_int64
_c_i32 = ctypes.c_int32
_c_int = ctypes.c_int
_ptr = ctypes.c_void_p
_size = ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/pccnn_b200.h one to one.
SIGNATURES = {
    "pccnn_last_error": (ctypes.c_char_p, []),
    "pccnn_version": (ctypes.c_char_p, []),
    "pccnn_check_status": (_c_int, [_c_int, _ptr]),
    "pccnn_validate_neighbors_workspace_bytes": (_size, []),
    "pccnn_validate_neighbors": (_c_int, [_c_i64, _c_i64, _ptr, _ptr, _c_i64, _ptr, _size, _ptr]),
    "pccnn_gemm_set_test_hooks": (_c_int, [_c_int, _c_int]),
    "pccnn_bounding_box": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_i64, _ptr, _ptr, _ptr]),
    "pccnn_grid_num_cells": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "pccnn_compute_keys": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "pccnn_sort_keys_workspace_bytes": (_size, [_c_i64]),
    "pccnn_sort_keys": (_c_int, [_c_i64, _ptr, _c_int, _ptr, _ptr, _c_int, _ptr, _ptr, _ptr, _size, _ptr]),
    "pccnn_grid_front_end_workspace_bytes": (_size, [_c_i64]),
    "pccnn_grid_front_end": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_i64, _ptr, _ptr, _ptr, _ptr,
                                      ctypes.POINTER(_c_i32), _ptr, _ptr, _ptr, _ptr, _ptr, _size, _ptr]),
    "pccnn_build_grid_ds": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_i64, _ptr, _ptr]),
    "pccnn_find_neighbors_workspace_bytes": (_size, [_c_int, _c_i64]),
    "pccnn_find_neighbors_min_workspace_bytes": (_size, [_c_int, _c_i64]),
    "pccnn_find_neighbors_count": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr,
                                            _c_i32, _c_i32, _ptr, ctypes.POINTER(_c_i64), _ptr, _size, _ptr]),
    "pccnn_find_neighbors_store": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr,
                                            _c_i32, _ptr, _ptr, _ptr, _ptr, _size, _ptr]),
    "pccnn_compute_pdf_workspace_bytes": (_size, [_c_int, _c_i64]),
    "pccnn_compute_pdf": (_c_int, [_c_int, _c_int, _ptr, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _size, _ptr]),
    "pccnn_compute_pdf_grads": (_c_int, [_c_int, _c_int, _ptr, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr]),
    "pccnn_compute_pdf_grads_symmetric": (_c_int, [_c_int, _c_int, _ptr, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _size,
                                                    _ptr]),
    "pccnn_poisson_disk_sampling_workspace_bytes": (_size, [_c_i64]),
    "pccnn_poisson_disk_sampling": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr,
                                             ctypes.POINTER(_c_i64), _ptr, _size, _ptr]),
    "pccnn_poisson_disk_sampling_grid_workspace_bytes": (_size, [_c_i64]),
    "pccnn_poisson_disk_sampling_grid": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
                                                  ctypes.POINTER(_c_i64), _ptr, _size, _ptr]),
    "pccnn_poisson_disk_sampling_static_max_points": (_c_i64, []),
    "pccnn_poisson_disk_sampling_static": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr,
                                                    ctypes.POINTER(_c_i64), _ptr]),
    "pccnn_conv_set_path": (_c_int, [_c_int]),
    "pccnn_conv_workspace_bytes": (_size, [_c_i64, _c_i64, _c_int, _c_int, _c_int]),
    "pccnn_kp_conv": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int,
                               ctypes.c_float, _ptr, _c_int, _ptr, _ptr, _size, _ptr]),
    "pccnn_kp_conv_grid_workspace_bytes": (_size, [_c_i64, _c_i64, _c_int, _c_int, _c_int]),
    "pccnn_kp_conv_grid": (_c_int, [_c_i64, _ptr, _ptr, _ptr, _ptr, _c_int, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
                                    _c_int, ctypes.c_float, _ptr, _c_int, _ptr, _ptr, _size, _ptr]),
    "pccnn_kp_conv_bf16": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int,
                                    ctypes.c_float, _ptr, _c_int, _ptr, _ptr, _size, _ptr]),
    "pccnn_mc_conv": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
                               _c_int, _c_int, _ptr, _c_int, _ptr, _ptr, _size, _ptr]),
    "pccnn_conv_grads_workspace_bytes": (_size, [_c_i64, _c_i64, _c_int, _c_int, _c_int]),
    "pccnn_conv_grads_set_weight_grads_event": (_c_int, [_ptr]),
    "pccnn_kp_conv_grads": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int,
                                     ctypes.c_float, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _size,
                                     _ptr]),
    "pccnn_mc_conv_grads": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr,
                                     _ptr, _c_int, _c_int, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr,
                                     _ptr, _size, _ptr]),
    "pccnn_conv_weight_var_workspace_bytes": (_size, [_c_i64, _c_i64, _c_int, _c_int]),
    "pccnn_kp_conv_weight_var": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int,
                                          ctypes.c_float, _ptr, _ptr, _size, _ptr]),
    "pccnn_mc_conv_weight_var": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr,
                                          _ptr, _c_int, _ptr, _ptr, _size, _ptr]),
    # density-normalised kernel-point convolutions: (D, n, pts, a, b, cin, m, samples, neighbors, ends, radii, kpts, K, sigma, ...)
    "pccnn_kp_conv_n": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int,
                                 ctypes.c_float, _ptr, _c_int, _ptr, _ptr, _size, _ptr]),
    "pccnn_kp_conv_n_grads": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int,
                                       ctypes.c_float, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _size, _ptr]),
    "pccnn_kp_conv_n_weight_var": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr,
                                            _c_int, ctypes.c_float, _ptr, _ptr, _size, _ptr]),
    "pccnn_pccnn_conv": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_int, _ptr, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int,
                                  ctypes.c_float, _ptr, _c_int, _ptr, _ptr, _size, _ptr]),
    "pccnn_pccnn_conv_grads": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_int, _ptr, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int,
                                        ctypes.c_float, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _size,
                                        _ptr]),
    "pccnn_pccnn_conv_weight_var": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_int, _ptr, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr,
                                             _c_int, ctypes.c_float, _ptr, _ptr, _size, _ptr]),
    "pccnn_sph_conv": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr, _c_int,
                                _ptr, _c_int, _ptr, _c_int, _ptr, _ptr, _size, _ptr]),
    "pccnn_sph_conv_grads": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr,
                                      _c_int, _ptr, _c_int, _ptr, _c_int, _ptr, _ptr, _ptr, _ptr, _size, _ptr]),
    "pccnn_sph_conv_weight_var": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int,
                                           _ptr, _c_int, _ptr, _c_int, _ptr, _ptr, _size, _ptr]),
    "pccnn_point_conv_basis": (_c_int, [_c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr]),
    "pccnn_point_conv_basis_grads": (_c_int, [_c_int, _c_i64, _c_i64, _c_i64, _ptr, _ptr, _ptr, _ptr, _ptr, _c_int, _ptr,
                                              _ptr, _ptr, _ptr, _ptr, _ptr]),
    "pccnn_point_conv": (_c_int, [_c_i64, _ptr, _c_int, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _c_int, _ptr, _ptr, _size,
                                  _ptr]),
    "pccnn_point_conv_grads": (_c_int, [_c_i64, _ptr, _c_int, _ptr, _c_int, _c_i64, _c_i64, _ptr, _ptr, _ptr, _c_int, _ptr,
                                        _ptr, _ptr, _ptr, _ptr, _size, _ptr]),
    "pccnn_point_conv_weight_var": (_c_int, [_c_i64, _ptr, _c_int, _ptr, _c_int, _c_i64, _ptr, _ptr, _ptr, _ptr, _size,
                                             _ptr]),
    "pccnn_gemm_workspace_bytes": (_size, [_c_i64, _c_int, _c_int]),
    "pccnn_gemm_f32": (_c_int, [_c_i64, _c_int, _c_int, _ptr, _c_i64, _ptr, _c_i64, _ptr, _c_i64, _c_int, _ptr,
                                _size, _ptr]),
    "pccnn_gemm_bf16": (_c_int, [_c_i64, _c_int, _c_int, _ptr, _ptr, _c_i64, _ptr, _ptr, _c_i64, _ptr, _c_i64, _ptr, _ptr]),
    "pccnn_gemm_tn_workspace_bytes": (_size, [_c_i64, _c_int, _c_int]),
    "pccnn_gemm_tn_f32": (_c_int, [_c_i64, _c_int, _c_int, _ptr, _c_i64, _ptr, _c_i64, _ptr, _c_i64, _c_int, _ptr,
                                   _size, _ptr]),
}


def library_path():
    return os.environ.get("PCCNN_B200_LIB", _build.LIB_PATH)


def _load():
    path = library_path()
    if not os.path.exists(path):
        # Source checkout without a built library: build it in place (needs nvcc).
        path = _build.build()
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error():
    return lib.pccnn_last_error().decode("utf-8", "replace")


def check(rc, what):
    if rc != 0:
        raise RuntimeError("%s failed (code %d): %s" % (what, rc, last_error()))
