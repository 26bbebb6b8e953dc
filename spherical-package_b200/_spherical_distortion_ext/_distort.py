"""Import-time stand-in for the reference's `_distort` module (lens-distortion sample maps, needs Eigen:
ext_modules/include/core/distortion.h).  Lens distortion is outside the mapped-operator path this package
rebuilds; the reference's `layers/functional/distortion.py:3` imports the module unconditionally, so the name must
resolve.  `DistortionType` is the real enum; everything else raises on use."""
from ._C import DistortionType  # noqa: F401


def create_distortion_sample_map(*args, **kwargs):
    raise ImportError("_spherical_distortion_ext._distort.create_distortion_sample_map is not provided by the B200 "
                      "mapped-operator package: build the reference's own `_distort` extension (it needs Eigen)")
