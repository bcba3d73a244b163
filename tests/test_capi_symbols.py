"""The C-ABI library builds, loads and exports every function declared in include/*.h.
No compute entry point is called here (there is no GPU on the machines that run this)."""
import ctypes
import glob
import os
import re

from conftest import ROOT


def declared_functions():
    names = []
    for header in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(header).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(pccnn_\w+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_hot_path():
    names = declared_functions()
    for needed in ["pccnn_compute_keys", "pccnn_build_grid_ds", "pccnn_find_neighbors_count",
                   "pccnn_find_neighbors_store", "pccnn_compute_pdf", "pccnn_compute_pdf_grads",
                   "pccnn_poisson_disk_sampling", "pccnn_sort_keys"]:
        assert needed in names


def test_library_exports_every_declared_symbol():
    from pccnn_lib_b200 import _build, _capi
    path = _build.build()
    lib = ctypes.CDLL(path)
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing
    # the ctypes table mirrors the header one to one
    assert sorted(_capi.SIGNATURES) == declared_functions()


def test_workspace_queries_and_argument_errors_need_no_gpu():
    from pccnn_lib_b200 import _capi
    lib = _capi.lib
    assert lib.pccnn_sort_keys_workspace_bytes(1000) > 8000
    assert lib.pccnn_find_neighbors_workspace_bytes(3, 1000) > 4000
    assert lib.pccnn_poisson_disk_sampling_workspace_bytes(1000) > 12000
    # invalid dimension is rejected before any CUDA call
    rc = lib.pccnn_compute_keys(9, 10, 1, 1, 1, 1, 1, 1, None)
    assert rc == 1 and "dimension" in _capi.last_error()
    assert lib.pccnn_version().startswith(b"pccnn_lib_b200")


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch
    from pccnn_lib_b200 import ops
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.compute_keys(torch.zeros(4, 3), torch.zeros(4, dtype=torch.int32), torch.zeros(1, 3),
                         torch.ones(3, dtype=torch.int32), torch.ones(3))
