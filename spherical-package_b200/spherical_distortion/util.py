"""Sample-map builders of the equirectangular kernels, evaluated on the GPU.

Same names, arguments and results as the reference's host-side builders
(layers/util/mapping_functions.py:44-163): a (ceil(H/stride), ceil(W/stride), kh*kw, 2) tensor of (x, y) pixel
coordinates.  The maps are produced directly in device memory (no host tensor algebra, no upload); `device` and
`dtype` say where and in which type."""
import torch

import _spherical_distortion_ext._C as _C


def _build(kind, shape, kernel_size, stride, dilation, device, dtype):
    like = torch.empty(0, device=device if device is not None else "cuda", dtype=dtype)
    return _C.build_kernel_map(shape[0], shape[1], kernel_size[0], kernel_size[1], stride, dilation, kind, like)


def grid_projection_map(shape, kernel_size, stride=1, dilation=1, device=None, dtype=torch.float32):
    """Kernel offsets taken on the latitude/longitude grid itself (no longitude wrap)."""
    return _build("grid", shape, kernel_size, stride, dilation, device, dtype)


def inverse_gnomonic_projection_map(shape, kernel_size, stride=1, dilation=1, device=None, dtype=torch.float32):
    """The kernel laid out on the tangent plane at every pixel and projected back onto the sphere."""
    return _build("inverse_gnomonic", shape, kernel_size, stride, dilation, device, dtype)


def inverse_equirectangular_projection_map(shape, kernel_size, stride=1, dilation=1, device=None, dtype=torch.float32):
    """Longitude offsets divided by cos(latitude) of the sampled row."""
    return _build("inverse_equirectangular", shape, kernel_size, stride, dilation, device, dtype)
