"""Compiles the UNMODIFIED reference extension (phermosilla/pccnn_lib, pccnn_lib_ops/*.cu + ops_list.cpp)
from where its sources lie into oracle/_ref/pccnn_lib_ops.so, for sm_100.  TEST INFRASTRUCTURE ONLY.

The reference's kernels are generic SIMT CUDA, so they run on a B200 once compiled for it.  The
result serves as a second checker next to the CPU oracle (tests/test_gpu_vs_reference_build.py):
same keys, tables and neighbor sets, convolution outputs within tolerance.  No reference source
is copied into this repository; only the built library lands in oracle/_ref/ (git-ignored).

Usage: python oracle/build_reference.py [/path/to/reference]   (about 10 minutes on 8 cores)
"""
import concurrent.futures
import glob
import os
import subprocess
import sys
import sysconfig


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
        "PCCNN_REFERENCE", os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference")))
    src_dir = os.path.join(ref, "pccnn_lib_ops")
    if not os.path.isdir(src_dir):
        print("reference sources not found at", src_dir)
        return 1
    from torch.utils import cpp_extension
    here = os.path.dirname(os.path.abspath(__file__))
    out_dir = os.path.join(here, "_ref")
    obj_dir = os.path.join(out_dir, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(src_dir, "**", "*.cu"), recursive=True)) + [os.path.join(src_dir, "ops_list.cpp")]
    includes = cpp_extension.include_paths("cuda") + [sysconfig.get_paths()["include"]]
    common = ["-DTORCH_EXTENSION_NAME=pccnn_lib_ops", "-DTORCH_API_INCLUDE_EXTENSION_H", "-std=c++17", "-O3"]
    for inc in includes:
        common += ["-isystem", inc]
    nvcc_flags = ["-gencode=arch=compute_100,code=sm_100", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
                  "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__",
                  "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-w"]

    def compile_one(src):
        obj = os.path.join(obj_dir, os.path.relpath(src, src_dir).replace(os.sep, "_") + ".o")
        if os.path.exists(obj) and os.path.getmtime(obj) > os.path.getmtime(src):
            return obj
        if src.endswith(".cu"):
            cmd = ["nvcc"] + common + nvcc_flags + ["-c", src, "-o", obj]
        else:
            cmd = ["/usr/bin/g++"] + common + ["-fPIC", "-w", "-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("failed: %s\n%s" % (" ".join(cmd), res.stderr[-3000:]))
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=int(os.environ.get("MAX_JOBS", "6"))) as ex:
        objs = list(ex.map(compile_one, sources))
    libs = []
    for d in cpp_extension.library_paths("cuda"):
        libs += ["-L" + d, "-Wl,-rpath," + d]
    out = os.path.join(out_dir, "pccnn_lib_ops.so")
    cmd = ["/usr/bin/g++", "-shared", "-o", out] + objs + libs + ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
                                                                  "-ltorch", "-ltorch_python", "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stderr[-3000:])
    print(out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
