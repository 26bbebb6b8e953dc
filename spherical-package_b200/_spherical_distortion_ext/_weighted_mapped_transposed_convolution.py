"""Weighted mapped transposed convolution (reference: ext_modules/include/layers/weighted_mapped_transposed_convolution_layer.h)."""
from ._C import (
    weighted_mapped_transposed_conv_forward,
    weighted_mapped_transposed_conv_backward,
)  # noqa: F401
