"""Mapped transposed convolution (reference: ext_modules/include/layers/mapped_transposed_convolution_layer.h)."""
from ._C import (
    mapped_transposed_conv_forward,
    mapped_transposed_conv_backward,
)  # noqa: F401
