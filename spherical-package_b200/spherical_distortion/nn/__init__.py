"""Modules of the mapped-operator path, with the constructor arguments,
parameter names/shapes and forward signatures of the reference
(layers/nn/mapped_convolution_layer.py:11-59,
layers/nn/mapped_transposed_convolution_layer.py:10-56,
layers/nn/mapped_max_pooling_layer.py:8-32, layers/nn/resample_layer.py:13-52),
so that existing state_dicts load unchanged.
"""
import math

import torch
import torch.nn as nn

from .. import functional as F
from ..layer_utils import InterpolationType


def _uniform_init(module, fan):
    bound = 1.0 / math.sqrt(fan)
    with torch.no_grad():
        module.weight.uniform_(-bound, bound)
        module.bias.uniform_(-bound, bound)


class MappedConvolution(nn.Module):
    """weight (out_channels, in_channels, kernel_size); output size = map size.  `activation="relu"` (an extension,
    default None = the reference's layer) fuses the activation into the convolution kernels."""

    def __init__(self, in_channels, out_channels, kernel_size=1, interpolation=InterpolationType.BILINEAR, bias=True,
                 activation=None):
        super().__init__()
        self.in_channels, self.out_channels, self.kernel_size, self.interp = in_channels, out_channels, kernel_size, interpolation
        self.activation = activation
        self.weight = nn.Parameter(torch.empty(out_channels, in_channels, kernel_size))
        self.bias = nn.Parameter(torch.empty(out_channels))
        self.reset_parameters()
        if not bias:
            self.bias = nn.Parameter(torch.zeros(out_channels))

    def reset_parameters(self):
        _uniform_init(self, self.in_channels * self.kernel_size)

    def forward(self, x, sample_map, interp_weights=None):
        return F.mapped_convolution(x, self.weight, self.bias, sample_map, self.kernel_size, self.interp, interp_weights,
                                    self.activation)


class MappedTransposedConvolution(nn.Module):
    """weight (in_channels, out_channels, kernel_size); the map has the input's size and points into the output."""

    def __init__(self, in_channels, out_channels, kernel_size=1, interpolation=InterpolationType.BILINEAR, bias=True):
        super().__init__()
        self.in_channels, self.out_channels, self.kernel_size, self.interp = in_channels, out_channels, kernel_size, interpolation
        self.weight = nn.Parameter(torch.empty(in_channels, out_channels, kernel_size))
        self.bias = nn.Parameter(torch.empty(out_channels))
        self.reset_parameters()
        if not bias:
            self.bias = nn.Parameter(torch.zeros(out_channels))

    def reset_parameters(self):
        _uniform_init(self, self.in_channels * self.kernel_size)

    def forward(self, x, oh, ow, sample_map, interp_weights=None):
        return F.mapped_transposed_convolution(x, self.weight, self.bias, sample_map, oh, ow, self.kernel_size,
                                               self.interp, interp_weights)


class MappedMaxPool(nn.Module):
    def __init__(self, kernel_size, interpolation=InterpolationType.BILINEAR, return_indices=False):
        super().__init__()
        self.kernel_size, self.interp, self.return_indices = kernel_size, interpolation, return_indices

    def forward(self, x, sample_map, interp_weights=None):
        pooled, idx_mask = F.mapped_max_pool(x, sample_map, self.kernel_size, self.interp, interp_weights)
        return (pooled, idx_mask) if self.return_indices else pooled


class Resample(nn.Module):
    """Scatter integer input positions to real-valued output positions."""

    def __init__(self, interpolation=InterpolationType.BILINEAR):
        super().__init__()
        self.interp = interpolation

    def forward(self, x, sample_map, output_shape, interp_weights=None):
        return F.resample(x, sample_map, output_shape, self.interp, interp_weights)


class Unresample(nn.Module):
    """Gather real-valued input positions to integer output positions."""

    def __init__(self, interpolation=InterpolationType.BILINEAR):
        super().__init__()
        self.interp = interpolation

    def forward(self, x, sample_map, interp_weights=None):
        return F.unresample(x, sample_map, self.interp, interp_weights)
