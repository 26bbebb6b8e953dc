"""Functional interface of the mapped-operator path.

Mirrors layers/functional/mapped_convolution.py:121-148,
layers/functional/mapped_pooling.py:203-245, layers/functional/resample.py:113-219,
layers/functional/convolution.py:62-71 and the map-driven halves of
layers/functional/tangent_images.py:6-55 of the reference: the same call
signatures and assertions, autograd Functions that hand the same positional
arguments to ``_spherical_distortion_ext`` (integers saved for backward travel
as 0-d tensors, the interpolation type as an int that is cast back to the
enum).
"""
import torch

import _spherical_distortion_ext._C as _C
import _spherical_distortion_ext._convolution as _std_conv
import _spherical_distortion_ext._mapped_avg_pooling as _avgpool
import _spherical_distortion_ext._mapped_convolution as _conv
import _spherical_distortion_ext._mapped_max_pooling as _pool
import _spherical_distortion_ext._mapped_transposed_convolution as _tconv
import _spherical_distortion_ext._resample as _res
import _spherical_distortion_ext._transposed_convolution as _std_tconv
import _spherical_distortion_ext._uv_resample as _uv
import _spherical_distortion_ext._voting_resample as _vote
import _spherical_distortion_ext._weighted_mapped_avg_pooling as _wavgpool
import _spherical_distortion_ext._weighted_mapped_convolution as _wconv
import _spherical_distortion_ext._weighted_mapped_max_pooling as _wpool
import _spherical_distortion_ext._weighted_mapped_transposed_convolution as _wtconv
import _spherical_distortion_ext._weighted_resample as _wres

from ..layer_utils import InterpolationType, check_args, check_input_map_shape


def _scalars(kernel_size, interp):
    return torch.tensor(kernel_size), torch.tensor(int(interp))


class _MappedConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, sample_map, kernel_size, interp, interp_weights):
        ctx.save_for_backward(x, weight, bias, sample_map, *_scalars(kernel_size, interp), interp_weights)
        if interp_weights is None:
            return _conv.mapped_conv_forward(x, sample_map, weight, bias, kernel_size, interp)
        return _wconv.weighted_mapped_conv_forward(x, sample_map, interp_weights, weight, bias, kernel_size, interp)

    @staticmethod
    def backward(ctx, grad_output):
        x, weight, bias, sample_map, kernel_size, interp, interp_weights = ctx.saved_tensors
        interp = InterpolationType(interp)
        if interp_weights is None:
            gx, gw, gb = _conv.mapped_conv_backward(grad_output, sample_map, x, weight, bias, kernel_size, interp)
        else:
            gx, gw, gb = _wconv.weighted_mapped_conv_backward(grad_output, sample_map, interp_weights, x, weight, bias,
                                                              kernel_size, interp)
        return gx, gw, gb, None, None, None, None


class _MappedConvReLU(torch.autograd.Function):
    """relu(mapped_convolution(...)) with the activation fused into the kernels; not in the reference."""

    @staticmethod
    def forward(ctx, x, weight, bias, sample_map, kernel_size, interp, interp_weights):
        out = _conv.mapped_conv_relu_forward(x, sample_map, interp_weights, weight, bias, kernel_size, interp)
        ctx.save_for_backward(x, weight, bias, sample_map, *_scalars(kernel_size, interp), interp_weights, out)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        x, weight, bias, sample_map, kernel_size, interp, interp_weights, out = ctx.saved_tensors
        gx, gw, gb = _conv.mapped_conv_relu_backward(grad_output, out, sample_map, interp_weights, x, weight, bias,
                                                     kernel_size, InterpolationType(interp))
        return gx, gw, gb, None, None, None, None


class _MappedTransposedConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, sample_map, oh, ow, kernel_size, interp, interp_weights):
        ctx.save_for_backward(x, sample_map, weight, bias, *_scalars(kernel_size, interp), interp_weights)
        if interp_weights is None:
            return _tconv.mapped_transposed_conv_forward(x, sample_map, weight, bias, oh, ow, kernel_size, interp)
        return _wtconv.weighted_mapped_transposed_conv_forward(x, sample_map, interp_weights, weight, bias, oh, ow,
                                                               kernel_size, interp)

    @staticmethod
    def backward(ctx, grad_output):
        x, sample_map, weight, bias, kernel_size, interp, interp_weights = ctx.saved_tensors
        interp = InterpolationType(interp)
        if interp_weights is None:
            gx, gw, gb = _tconv.mapped_transposed_conv_backward(grad_output, sample_map, x, weight, bias, kernel_size,
                                                                interp)
        else:
            gx, gw, gb = _wtconv.weighted_mapped_transposed_conv_backward(grad_output, sample_map, interp_weights, x,
                                                                          weight, bias, kernel_size, interp)
        return gx, gw, gb, None, None, None, None, None, None


class _MappedMaxPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, sample_map, kernel_size, interp, interp_weights):
        if interp_weights is None:
            pooled, idx_mask = _pool.mapped_max_pool(x, sample_map, kernel_size, interp)
        else:
            pooled, idx_mask = _wpool.weighted_mapped_max_pool(x, sample_map, interp_weights, kernel_size, interp)
        ctx.mark_non_differentiable(idx_mask)
        ctx.save_for_backward(torch.tensor([x.shape[2], x.shape[3]]), idx_mask, sample_map,
                              *_scalars(kernel_size, interp), interp_weights)
        return pooled, idx_mask

    @staticmethod
    def backward(ctx, grad_output, _idx_grad=None):
        in_shape, idx_mask, sample_map, kernel_size, interp, interp_weights = ctx.saved_tensors
        interp = InterpolationType(interp)
        if interp_weights is None:
            gx = _pool.mapped_max_unpool(grad_output, idx_mask, sample_map, in_shape[0], in_shape[1], kernel_size, interp)
        else:
            gx = _wpool.weighted_mapped_max_unpool(grad_output, idx_mask, sample_map, interp_weights, in_shape[0],
                                                   in_shape[1], kernel_size, interp)
        return gx, None, None, None, None


class _Resample(torch.autograd.Function):
    """Scatter forward, gather backward (layers/functional/resample.py:11-48)."""

    @staticmethod
    def forward(ctx, x, sample_map, output_shape, interp, interp_weights):
        ctx.save_for_backward(sample_map, torch.tensor(int(interp)), interp_weights)
        if interp_weights is None:
            return _res.resample_to_map(x, sample_map, output_shape[0], output_shape[1], interp)
        return _wres.weighted_resample_to_map(x, sample_map, interp_weights, output_shape[0], output_shape[1], interp)

    @staticmethod
    def backward(ctx, grad_output):
        sample_map, interp, interp_weights = ctx.saved_tensors
        interp = InterpolationType(interp)
        grad_output = grad_output.contiguous()
        if interp_weights is None:
            return _res.resample_from_map(grad_output, sample_map, interp), None, None, None, None
        return _wres.weighted_resample_from_map(grad_output, sample_map, interp_weights, interp), None, None, None, None


class _Unresample(torch.autograd.Function):
    """Gather forward, scatter backward (layers/functional/resample.py:51-83)."""

    @staticmethod
    def forward(ctx, x, sample_map, interp, interp_weights):
        ctx.save_for_backward(sample_map, torch.tensor(int(interp)), interp_weights)
        ctx.in_hw = (x.shape[2], x.shape[3])
        if interp_weights is None:
            return _res.resample_from_map(x, sample_map, interp)
        return _wres.weighted_resample_from_map(x, sample_map, interp_weights, interp)

    @staticmethod
    def backward(ctx, grad_output):
        sample_map, interp, interp_weights = ctx.saved_tensors
        interp = InterpolationType(interp)
        grad_output = grad_output.contiguous()
        h, w = ctx.in_hw
        if interp_weights is None:
            return _res.resample_to_map(grad_output, sample_map, h, w, interp), None, None, None
        return _wres.weighted_resample_to_map(grad_output, sample_map, interp_weights, h, w, interp), None, None, None


def mapped_convolution(input, weight, bias, sample_map, kernel_size, interp, interp_weights=None, activation=None):
    """`activation` (None or "relu") is an extension of this library: the ReLU runs inside the convolution kernels
    instead of as separate passes over the output and its gradient."""
    check_args(input, sample_map, interp_weights, weight.shape[1], weight.shape[2])
    assert activation in (None, "relu"), "activation must be None or 'relu'"
    fn = _MappedConvReLU if activation == "relu" else _MappedConv
    return fn.apply(input, weight, bias, sample_map, kernel_size, interp, interp_weights)


def mapped_transposed_convolution(input, weight, bias, sample_map, output_height, output_width, kernel_size, interp,
                                  interp_weights=None):
    check_args(input, sample_map, interp_weights, weight.shape[0], weight.shape[2])
    check_input_map_shape(input, sample_map)
    return _MappedTransposedConv.apply(input, weight, bias, sample_map, output_height, output_width, kernel_size,
                                       interp, interp_weights)


def mapped_max_pool(input, sample_map, kernel_size, interp, interp_weights=None):
    check_args(input, sample_map, interp_weights, None, kernel_size)
    return _MappedMaxPool.apply(input, sample_map, kernel_size, interp, interp_weights)


def _with_batch(fn, input, *args):
    assert input.dim() in (3, 4), "Input must have 3 or 4 dimensions (input.dim() == {})".format(input.dim())
    if input.dim() == 3:
        return fn(input.unsqueeze(0), *args).squeeze(0)
    return fn(input, *args)


def resample(input, sample_map, output_shape, interp, interp_weights=None):
    def run(x):
        check_args(x, sample_map, interp_weights, None, None)
        check_input_map_shape(x, sample_map)
        return _Resample.apply(x, sample_map, output_shape, interp, interp_weights)
    return _with_batch(run, input)


def unresample(input, sample_map, interp, interp_weights=None):
    def run(x):
        check_args(x, sample_map, interp_weights, None, None)
        return _Unresample.apply(x, sample_map, interp, interp_weights)
    return _with_batch(run, input)


# ---- average pooling (layers/functional/mapped_pooling.py:9-101, 203-223) ---------------------------------
class _MappedAvgPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, sample_map, kernel_size, interp, interp_weights):
        ctx.save_for_backward(torch.tensor([x.shape[2], x.shape[3]]), sample_map, *_scalars(kernel_size, interp), interp_weights)
        if interp_weights is None:
            return _avgpool.mapped_avg_pool(x, sample_map, kernel_size, interp)
        return _wavgpool.weighted_mapped_avg_pool(x, sample_map, interp_weights, kernel_size, interp)

    @staticmethod
    def backward(ctx, grad_output):
        in_shape, sample_map, kernel_size, interp, interp_weights = ctx.saved_tensors
        interp = InterpolationType(interp)
        if interp_weights is None:
            gx = _avgpool.mapped_avg_unpool(grad_output, sample_map, in_shape[0], in_shape[1], kernel_size, interp)
        else:
            gx = _wavgpool.weighted_mapped_avg_unpool(grad_output, sample_map, interp_weights, in_shape[0], in_shape[1],
                                                      kernel_size, interp)
        return gx, None, None, None, None


class _MappedAvgUnpool(torch.autograd.Function):
    """The adjoint used as a forward operator (an up-sampling layer); its gradient is the pooling itself."""

    @staticmethod
    def forward(ctx, x, oh, ow, sample_map, kernel_size, interp, interp_weights):
        ctx.save_for_backward(sample_map, *_scalars(kernel_size, interp), interp_weights)
        if interp_weights is None:
            return _avgpool.mapped_avg_unpool(x, sample_map, oh, ow, kernel_size, interp)
        return _wavgpool.weighted_mapped_avg_unpool(x, sample_map, interp_weights, oh, ow, kernel_size, interp)

    @staticmethod
    def backward(ctx, grad_output):
        sample_map, kernel_size, interp, interp_weights = ctx.saved_tensors
        interp = InterpolationType(interp)
        grad_output = grad_output.contiguous()
        if interp_weights is None:
            gx = _avgpool.mapped_avg_pool(grad_output, sample_map, kernel_size, interp)
        else:
            gx = _wavgpool.weighted_mapped_avg_pool(grad_output, sample_map, interp_weights, kernel_size, interp)
        return gx, None, None, None, None, None, None


def mapped_avg_pool(input, sample_map, kernel_size, interp, interp_weights=None):
    check_args(input, sample_map, interp_weights, None, kernel_size)
    return _MappedAvgPool.apply(input, sample_map, kernel_size, interp, interp_weights)


def mapped_avg_unpool(input, oh, ow, sample_map, kernel_size, interp, interp_weights=None):
    check_args(input, sample_map, interp_weights, None, kernel_size)
    check_input_map_shape(input, sample_map)
    return _MappedAvgUnpool.apply(input, oh, ow, sample_map, kernel_size, interp, interp_weights)


# ---- UV-map and voting resampling (layers/functional/resample.py:86-110, 159-219) -----------------------------
class _UVResample(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, quad_idx, tex_uv, interp):
        ctx.save_for_backward(quad_idx, tex_uv, torch.tensor(int(interp)), torch.tensor(x.shape[-3:]))
        return _uv.resample_from_uv_maps(x, quad_idx, tex_uv, interp)

    @staticmethod
    def backward(ctx, grad_output):
        quad_idx, tex_uv, interp, tex_shape = ctx.saved_tensors
        return _uv.resample_to_uv_maps(grad_output.contiguous(), quad_idx, tex_uv, tex_shape[0], tex_shape[1], tex_shape[2],
                                       InterpolationType(interp)), None, None, None


def uv_resample(input, quad_idx, tex_uv, interp):
    """input ([B,] C, textures, TH, TW) -> ([B,] C, H, W): every image pixel samples texture quad_idx[y, x] at tex_uv[y, x]."""
    assert input.dim() in (4, 5), "Input must have 4 or 5 dimensions (input.dim() == {})".format(input.dim())
    if input.dim() == 4:
        return _UVResample.apply(input.unsqueeze(0), quad_idx, tex_uv, interp).squeeze(0)
    return _UVResample.apply(input, quad_idx, tex_uv, interp)


def voting_resample(input, sample_map, interp_weights, output_shape, num_candidates):
    """Integer labels are moved through an integer (x, y) sample map; every output pixel takes the label most of the
    pixels that land on it carry (layers/functional/resample.py:159-190; `interp_weights` is accepted and, as in the
    reference, has no effect on the result)."""
    def run(x):
        check_args(x, sample_map, interp_weights, None, None)
        check_input_map_shape(x, sample_map)
        return _vote.voting_resample_to_map(x.long().contiguous(), sample_map.long().contiguous(), *output_shape, num_candidates)
    return _with_batch(run, input)


def resample_normalized(input, sample_map, output_shape, interp, interp_weights=None):
    """resample(...) divided by the resampled weight sum: scatter(x) / (scatter(1) + 1e-12), the normalisation the
    reference applies after its scatters (layers/functional/sphere_ops.py:74-80), fused into the scatter kernel.
    Forward only (no autograd node)."""
    def run(x):
        check_args(x, sample_map, interp_weights, None, None)
        check_input_map_shape(x, sample_map)
        return _C.resample_to_map_normalized(x, sample_map, interp_weights, output_shape[0], output_shape[1], interp)
    return _with_batch(run, input.detach())


# ---- tangent images (layers/functional/tangent_images.py:6-55) -------------------------------------------------
def create_tangent_images(input, sample_map, num_samples, interpolation=InterpolationType.BISPHERICAL):
    """([B,] C, H, W) equirectangular image -> ([B,] C, faces, num_samples, num_samples) tangent images through a
    (faces, num_samples*num_samples, 2) sample map.  The reference derives the map from its icosphere mesh utilities
    (layers/util/tangent_images.py), which are outside this package: pass the map in."""
    t = unresample(input, sample_map, interpolation)
    return t.view(*t.shape[:-1], num_samples, num_samples)


def tangent_images_to_equirectangular(tangent_images, quad, uv, interpolation=InterpolationType.BILINEAR):
    """([B,] C, faces, D, D) tangent images -> ([B,] C, H, W) through the (H, W) face-index / (H, W, 2) UV maps."""
    assert tangent_images.dim() in (4, 5), \
        "tangent_images must be a 4D or 5D tensor (tangent_images.dim() == {})".format(tangent_images.dim())
    return uv_resample(tangent_images, quad, uv, interpolation)


# ---- standard convolution (layers/functional/convolution.py:10-71) -------------------------------------------
class _Convolution(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, kernel_size, stride, padding, dilation):
        ctx.save_for_backward(x, weight, bias)
        ctx.geom = (tuple(kernel_size), tuple(stride), tuple(padding), tuple(dilation))
        return _std_conv.conv_forward(x, weight, bias, *kernel_size, *stride, *padding, *dilation)

    @staticmethod
    def backward(ctx, grad_output):
        x, weight, bias = ctx.saved_tensors
        k, s, p, d = ctx.geom
        gx, gw, gb = _std_conv.conv_backward(grad_output, x, weight, bias, *k, *s, *p, *d)
        return gx, gw, gb, None, None, None, None


class _TransposedConvolution(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, kernel_size, stride, padding, dilation):
        ctx.save_for_backward(x, weight, bias)
        ctx.geom = (tuple(kernel_size), tuple(stride), tuple(padding), tuple(dilation))
        return _std_tconv.transposed_conv_forward(x, weight, bias, *kernel_size, *stride, *padding, *dilation)

    @staticmethod
    def backward(ctx, grad_output):
        x, weight, bias = ctx.saved_tensors
        k, s, p, d = ctx.geom
        gx, gw, gb = _std_tconv.transposed_conv_backward(grad_output, x, weight, bias, *k, *s, *p, *d)
        return gx, gw, gb, None, None, None, None


def convolution(input, weight, bias, kernel_size, stride, padding, dilation):
    return _Convolution.apply(input, weight, bias, kernel_size, stride, padding, dilation)


def transposed_convolution(input, weight, bias, kernel_size, stride, padding, dilation):
    return _TransposedConvolution.apply(input, weight, bias, kernel_size, stride, padding, dilation)
