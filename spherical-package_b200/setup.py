"""Build the native parts in-tree:  python setup.py build_ext --inplace

`build_ext` compiles csrc/*.cu for sm_100a into libsphmap.so (the C ABI of include/sphmap.h) and
csrc/torch_shim.cpp into the PyTorch host extension `_spherical_distortion_ext._C`; see build.py.
The packages are `_spherical_distortion_ext` (the drop-in for the reference's native package),
`spherical_distortion` (mirror of the reference's Python layer for the mapped-operator path) and `sphmap`.
"""
import os
import sys

from setuptools import Command, setup

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import build as native_build  # noqa: E402


class BuildNative(Command):
    description = "compile libsphmap.so (nvcc, sm_100a) and the torch host extension"
    user_options = [("inplace", "i", "ignored: the native build is always in-tree")]

    def initialize_options(self):
        self.inplace = 1

    def finalize_options(self):
        pass

    def run(self):
        native_build.build_all(verbose=True)


setup(
    name="spherical-mapped-ops-b200",
    version="1.0.0",
    packages=["_spherical_distortion_ext", "spherical_distortion", "spherical_distortion.nn",
              "spherical_distortion.functional", "sphmap"],
    package_data={"_spherical_distortion_ext": ["*.so"]},
    cmdclass={"build_ext": BuildNative},
)
