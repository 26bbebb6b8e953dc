"""Build the native parts of the package in-tree.

    python build.py            # libsphmap.so (nvcc, sm_100a) + the PyTorch host extension (_C)
    python build.py --lib-only # only the C-ABI library (no torch headers needed)
    python build.py --checked  # also libsphmap_checked.so: same ABI, every data-dependent index range-checked

Outputs go next to the Python modules in ``_spherical_distortion_ext/``:
``libsphmap.so`` (the C ABI of include/sphmap.h; depends only on the CUDA
runtime) and ``_C.<abi>.so`` (pybind11 host shim, links libsphmap.so and torch).
nvcc cross-compiles for sm_100a, so no GPU is needed to build.
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "_spherical_distortion_ext")
OBJ = os.path.join(HERE, "build", "obj")
INCLUDE = os.path.join(ROOT, "include")

CU_SOURCES = ["resample.cu", "plan.cu", "pool.cu", "maps.cu", "conv.cu", "conv_simt.cu", "conv_small.cu", "conv_tc.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--extended-lambda",
              "-Xcompiler", "-fPIC", "-I" + INCLUDE, "-I" + CSRC]
# extra compiler flags for developer builds, e.g. SPHMAP_NVCC_FLAGS="-DSPH_TC_TIMING" (per-role cycle counters)
NVCC_FLAGS += os.environ.get("SPHMAP_NVCC_FLAGS", "").split()


def _nvcc():
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout[-3000:], r.stderr[-6000:]))
    return r.stdout + r.stderr


def build_lib(verbose=False, ptxas_info=False, checked=False):
    """libsphmap.so, or with checked=True libsphmap_checked.so: the same sources compiled with -DSPH_BOUNDS_CHECK
    (every data-dependent index is range-checked on the device; see include/sphmap.h)."""
    obj_dir = OBJ + ("_checked" if checked else "")
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))] + \
              [os.path.join(INCLUDE, "sphmap.h")]
    logs = []

    def one(src):
        s, o = os.path.join(CSRC, src), os.path.join(obj_dir, src[:-3] + ".o")
        if _newer(o, [s] + headers):
            return o
        flags = NVCC_FLAGS + (["-DSPH_BOUNDS_CHECK"] if checked else []) + (["-Xptxas", "-v"] if ptxas_info else [])
        logs.append(_run([_nvcc()] + flags + ["-c", s, "-o", o]))
        return o

    with ThreadPoolExecutor(len(CU_SOURCES)) as ex:
        objs = list(ex.map(one, CU_SOURCES))
    lib = os.path.join(OUT, "libsphmap_checked.so" if checked else "libsphmap.so")
    if not _newer(lib, objs):
        _run([_nvcc(), "-shared", "-o", lib] + objs + ["-lcudart"])
    if verbose:
        print("built", lib)
    return lib, "".join(logs)


def build_ext(verbose=False):
    import torch
    from torch.utils import cpp_extension as ce

    src = os.path.join(CSRC, "torch_shim.cpp")
    out = os.path.join(OUT, "_C" + sysconfig.get_config_var("EXT_SUFFIX"))
    if _newer(out, [src, os.path.join(INCLUDE, "sphmap.h")]):
        return out
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = [cxx, "-shared", "-fPIC", "-std=c++17", "-O2", "-w", "-DTORCH_EXTENSION_NAME=_C",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI)),
           "-I" + INCLUDE]
    for i in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]:
        cmd += ["-isystem", i]
    cmd += [src, "-o", out, "-L" + OUT, "-lsphmap", "-Wl,-rpath,$ORIGIN"]
    for lp in ce.library_paths():
        cmd += ["-L" + lp, "-Wl,-rpath," + lp]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-L" + os.path.join(cuda_home, "lib64"), "-lcudart"]
    _run(cmd)
    if verbose:
        print("built", out)
    return out


def build_all(verbose=False):
    build_lib(verbose)
    build_lib(verbose, checked=True)
    build_ext(verbose)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--lib-only", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / shared memory per kernel")
    ap.add_argument("--checked", action="store_true", help="also build libsphmap_checked.so (-DSPH_BOUNDS_CHECK)")
    a = ap.parse_args()
    lib, log = build_lib(True, a.ptxas_info)
    if a.checked:
        build_lib(True, False, checked=True)
    if a.ptxas_info:
        print(log)
    if not a.lib_only:
        build_ext(True)
    sys.exit(0)
