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


def test_ctypes_signatures_match_the_header_argument_by_argument():
    """Every prototype of include/*.h against the ctypes table: same number of arguments and the same kind
    (pointer / int / int32 / int64 / size_t / float) at every position, and the same return type."""
    from pccnn_lib_b200 import _capi
    text = ""
    for header in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text += re.sub(r"/\*.*?\*/", "", open(header).read(), flags=re.S)

    def kind_of_c(decl):
        decl = decl.strip()
        if "*" in decl:
            return "ptr"
        base = decl.replace("const", "").split()
        base = base[0] if len(base) == 1 else " ".join(base[:-1])
        return {"int": "int", "int32_t": "i32", "int64_t": "i64", "size_t": "size", "float": "float", "void": "void"}[base.strip()]

    def kind_of_ctype(t):
        if t in (ctypes.c_void_p, ctypes.c_char_p) or (isinstance(t, type) and issubclass(t, ctypes._Pointer)):
            return "ptr"
        return {ctypes.c_int: "int", ctypes.c_int32: "i32", ctypes.c_int64: "i64", ctypes.c_size_t: "size",
                ctypes.c_float: "float"}[t]

    protos = re.findall(r"([\w\s\*]+?)\b(pccnn_\w+)\s*\(([^)]*)\)\s*;", text)
    assert len(protos) == len(_capi.SIGNATURES)
    for ret, name, args in protos:
        res, argtypes = _capi.SIGNATURES[name]
        c_args = [] if args.strip() in ("", "void") else [kind_of_c(a) for a in args.split(",")]
        py_args = [kind_of_ctype(t) for t in argtypes]
        # on this ABI int and int32_t are the same type; the table may use either
        norm = lambda ks: ["int" if k == "i32" else k for k in ks]
        assert norm(c_args) == norm(py_args), (name, c_args, py_args)
        ret_kind = "ptr" if "*" in ret else kind_of_c(ret + " x")
        assert norm([ret_kind]) == norm(["ptr" if res == ctypes.c_char_p else kind_of_ctype(res)]), name
