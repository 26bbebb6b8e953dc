"""Mapped convolution (reference: ext_modules/include/layers/mapped_convolution_layer.h:138-143)."""
from ._C import (
    mapped_conv_forward,
    mapped_conv_backward,
)  # noqa: F401
