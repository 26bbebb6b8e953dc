"""Modules of the mapped-operator path, with the constructor arguments,
parameter names/shapes and forward signatures of the reference
(layers/nn/mapped_convolution_layer.py:11-59,
layers/nn/mapped_transposed_convolution_layer.py:10-56,
layers/nn/mapped_max_pooling_layer.py:8-32, layers/nn/mapped_avg_pooling_layer.py:7-46,
layers/nn/resample_layer.py:13-87, layers/nn/convolution_layer.py:10-52,
layers/nn/transposed_convolution_layer.py:10-56), so that existing state_dicts load unchanged.
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


class MappedAvgPool(nn.Module):
    def __init__(self, kernel_size, interpolation=InterpolationType.BILINEAR):
        super().__init__()
        self.kernel_size, self.interp = kernel_size, interpolation

    def forward(self, x, sample_map, interp_weights=None):
        return F.mapped_avg_pool(x, sample_map, self.kernel_size, self.interp, interp_weights)


class MappedAvgUnpool(nn.Module):
    """x (B, C, IH, IW) with a map of its own size pointing into the (oh, ow) output."""

    def __init__(self, kernel_size, interpolation=InterpolationType.BILINEAR):
        super().__init__()
        self.kernel_size, self.interp = kernel_size, interpolation

    def forward(self, x, oh, ow, sample_map, interp_weights=None):
        return F.mapped_avg_unpool(x, oh, ow, sample_map, self.kernel_size, self.interp, interp_weights)


class ResampleFromUV(nn.Module):
    """Gathers an image from N textures: x (B, C, N, TH, TW), quad_idx (H, W) int64, tex_uv (H, W, 2)."""

    def __init__(self, interpolation=InterpolationType.BILINEAR):
        super().__init__()
        assert interpolation in [InterpolationType.NEAREST, InterpolationType.BILINEAR], "Unsupported interpolation type"
        self.interp = interpolation

    def forward(self, x, quad_idx, tex_uv):
        assert x.dim() == 5, "Input expected to be 5 dimensional tensor ({} != {})".format(x.dim(), 5)
        assert quad_idx.dim() == 2 and quad_idx.dtype == torch.int64, "quad_idx expected to be 2 dimension tensor of type long"
        assert tex_uv.shape[:2] == quad_idx.shape, \
            "tex_uv expected to have same first two dimensions as quad_idx ({} != {})".format(tex_uv.shape[:2], quad_idx.shape)
        return F.uv_resample(x, quad_idx, tex_uv, self.interp)


def _pair(v):
    return tuple(v) if isinstance(v, (tuple, list)) else (v, v)


class _StandardConv(nn.Module):
    transposed = False

    def __init__(self, in_channels, out_channels, kernel_size=1, stride=1, padding=0, dilation=1):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding, self.dilation = _pair(kernel_size), _pair(stride), _pair(padding), _pair(dilation)
        shape = (in_channels, out_channels) if self.transposed else (out_channels, in_channels)
        self.weight = nn.Parameter(torch.empty(*shape, *self.kernel_size))
        self.bias = nn.Parameter(torch.empty(out_channels))
        _uniform_init(self, in_channels * self.kernel_size[0] * self.kernel_size[1])


class Convolution(_StandardConv):
    """Plain 2-D convolution with the reference layer's parameters: weight (out, in, kh, kw)."""

    def forward(self, x):
        return F.convolution(x, self.weight, self.bias, self.kernel_size, self.stride, self.padding, self.dilation)


class TransposedConvolution(_StandardConv):
    """Plain 2-D transposed convolution: weight (in, out, kh, kw)."""
    transposed = True

    def forward(self, x):
        return F.transposed_convolution(x, self.weight, self.bias, self.kernel_size, self.stride, self.padding, self.dilation)
