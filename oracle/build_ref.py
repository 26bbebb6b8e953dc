"""Build the reference's own CPU extension modules for the mapped-operator path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this file or
anything it builds.  Only the parity tests, the smoke check and the CPU-baseline
leg of the benchmark may load what is built here.

The reference checkout (``ext_modules/src/cpp/*.cpp`` + ``ext_modules/include``)
is compiled *where it lies* with the flags of the reference's ``setup.py``
(``-fopenmp -O3 -D__NO_CUDA__``, setup.py:42,54); no reference source is copied.
The shared objects land in ``oracle/_ref/_spherical_distortion_ext/`` (a
git-ignored folder) under the module names of setup.py:62-195, so that
``oracle/ref.py`` can import them as the package the reference's Python layer
expects.

Usage:  python oracle/build_ref.py [--reference /path/to/Spherical-Package] [-j N]
(the default is $SPHERICAL_PACKAGE_REFERENCE, else the folder `reference` beside this repository)
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "_spherical_distortion_ext")

# module name -> source basename (setup.py:62-195 of the reference)
MODULES = {
    "_enums": "enum_export",
    "_resample": "resample_layer",
    "_weighted_resample": "weighted_resample_layer",
    "_mapped_convolution": "mapped_convolution_layer",
    "_weighted_mapped_convolution": "weighted_mapped_convolution_layer",
    "_mapped_transposed_convolution": "mapped_transposed_convolution_layer",
    "_weighted_mapped_transposed_convolution": "weighted_mapped_transposed_convolution_layer",
    "_mapped_max_pooling": "mapped_max_pooling_layer",
    "_weighted_mapped_max_pooling": "weighted_mapped_max_pooling_layer",
    "_mapped_avg_pooling": "mapped_avg_pooling_layer",
    "_weighted_mapped_avg_pooling": "weighted_mapped_avg_pooling_layer",
    "_uv_resample": "uv_resample_layer",
    "_voting_resample": "voting_resample_layer",
    "_convolution": "convolution_layer",
    "_transposed_convolution": "transposed_convolution_layer",
}


def _compile(ref, name, base, cxx):
    import torch
    from torch.utils import cpp_extension as ce

    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    out = os.path.join(OUT, name + suffix)
    src = os.path.join(ref, "ext_modules", "src", "cpp", base + ".cpp")
    if os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return name, "cached"
    inc = [os.path.join(ref, "ext_modules", "include")] + ce.include_paths() + [sysconfig.get_paths()["include"]]
    cmd = [cxx, "-shared", "-fPIC", "-std=c++17", "-O3", "-fopenmp", "-D__NO_CUDA__",
           "-DTORCH_EXTENSION_NAME=" + name, "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI)), "-w"]
    for i in inc:
        cmd += ["-isystem", i]
    cmd += [src, "-o", out]
    for lp in ce.library_paths():
        cmd += ["-L" + lp, "-Wl,-rpath," + lp]
    cmd += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-fopenmp"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building %s failed:\n%s" % (name, r.stderr[-4000:]))
    return name, "built"


def default_reference():
    """Where the reference checkout is looked for: $SPHERICAL_PACKAGE_REFERENCE, else a folder named `reference`
    beside this repository."""
    return os.environ.get("SPHERICAL_PACKAGE_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(reference=None, jobs=4, quiet=False):
    """Compile every module of MODULES; returns the output directory."""
    reference = reference or default_reference()
    if not os.path.isdir(os.path.join(reference, "ext_modules")):
        raise FileNotFoundError("reference checkout not found at " + reference)
    os.makedirs(OUT, exist_ok=True)
    init = os.path.join(OUT, "__init__.py")
    if not os.path.exists(init):
        open(init, "w").close()
    # /usr/bin/g++ links OpenMP; a wrapper compiler earlier on PATH may not.
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    with ThreadPoolExecutor(jobs) as ex:
        for name, how in ex.map(lambda kv: _compile(reference, kv[0], kv[1], cxx), MODULES.items()):
            if not quiet:
                print("oracle/_ref: %-44s %s" % (name, how))
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference())
    ap.add_argument("-j", type=int, default=4)
    a = ap.parse_args()
    build(a.reference, a.j)
    sys.exit(0)
