"""Functional interface of the mapped-operator path.

Mirrors layers/functional/mapped_convolution.py:121-148,
layers/functional/mapped_pooling.py:225-232 and layers/functional/resample.py:113-157
of the reference: the same call signatures and assertions, autograd Functions
that hand the same positional arguments to ``_spherical_distortion_ext``
(integers saved for backward travel as 0-d tensors, the interpolation type as
an int that is cast back to the enum).
"""
import torch

import _spherical_distortion_ext._mapped_convolution as _conv
import _spherical_distortion_ext._mapped_max_pooling as _pool
import _spherical_distortion_ext._mapped_transposed_convolution as _tconv
import _spherical_distortion_ext._resample as _res
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
