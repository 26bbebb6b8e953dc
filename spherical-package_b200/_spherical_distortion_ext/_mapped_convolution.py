"""Mapped convolution (reference: ext_modules/include/layers/mapped_convolution_layer.h:138-143), plus the
fused-ReLU variants of this library (no reference counterpart)."""
from ._C import (
    mapped_conv_forward,
    mapped_conv_backward,
    mapped_conv_relu_forward,
    mapped_conv_relu_backward,
)  # noqa: F401
