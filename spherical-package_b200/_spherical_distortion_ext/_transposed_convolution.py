"""Same module name and functions as the reference's `_transposed_convolution` (ext_modules/include/layers/transposed_convolution_layer.h:145-150)."""
from ._C import transposed_conv_forward, transposed_conv_backward  # noqa: F401
