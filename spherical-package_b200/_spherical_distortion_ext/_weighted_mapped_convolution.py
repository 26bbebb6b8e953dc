"""Weighted mapped convolution (reference: ext_modules/include/layers/weighted_mapped_convolution_layer.h)."""
from ._C import (
    weighted_mapped_conv_forward,
    weighted_mapped_conv_backward,
)  # noqa: F401
