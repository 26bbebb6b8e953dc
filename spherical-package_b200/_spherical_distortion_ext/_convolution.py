"""Same module name and functions as the reference's `_convolution` (ext_modules/include/layers/convolution_layer.h:134-137)."""
from ._C import conv_forward, conv_backward  # noqa: F401
