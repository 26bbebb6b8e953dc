"""The reference's own layer tests, re-run on the GPU through the mirror `spherical_distortion.nn` modules: each
known-answer case of the reference suite (inputs and hand-computed outputs from tests/golden/reference_kats.pt) goes
through the nn.Module, its output is compared with the hand-computed tensor, `backward` runs, and
`torch.autograd.gradcheck` validates the backward kernels in float64, exactly as the reference's tests/utils.py does."""
import os

import pytest
import torch
from torch.autograd import gradcheck

pytestmark = pytest.mark.gpu


def _kats(golden_dir):
    return torch.load(os.path.join(golden_dir, "reference_kats.pt"), weights_only=False)


def _layer(c):
    from spherical_distortion.nn import (InterpolationType, MappedConvolution, MappedMaxPool,
                                         MappedTransposedConvolution, Unresample)
    it = InterpolationType(c["interp"])
    if c["op"] == "conv":
        co, ci, k = c["weight"].shape
        layer = MappedConvolution(ci, co, k, it).double().cuda()
    elif c["op"] == "tconv":
        ci, co, k = c["weight"].shape
        layer = MappedTransposedConvolution(ci, co, k, it).double().cuda()
    elif c["op"] == "pool":
        return MappedMaxPool(c["kernel_size"], it).double().cuda()
    else:
        return Unresample(it).cuda()
    with torch.no_grad():
        layer.weight.copy_(c["weight"])
        layer.bias.copy_(c["bias"])
    return layer


def test_reference_layer_tests_forward_backward_and_gradcheck(golden_dir):
    n = 0
    for c in _kats(golden_dir):
        layer = _layer(c)
        x = c["input"].clone().cuda().requires_grad_(True)
        m = c["sample_map"].cuda()
        iw = c["interp_weights"].cuda() if c.get("interp_weights") is not None else None
        args = (x, c["oh"], c["ow"], m, iw) if c["op"] == "tconv" else (x, m, iw)
        out = layer(*args)
        exp = c["expected"].to(out.dtype).cuda().expand_as(out)
        torch.testing.assert_close(out, exp, rtol=1e-7, atol=1e-9, msg=c["name"])
        out.backward(torch.ones_like(out))
        torch.testing.assert_close(x.grad.cpu(), c["ref_grads"][0], rtol=1e-12, atol=1e-12, msg=c["name"])
        if c["op"] in ("conv", "tconv"):
            torch.testing.assert_close(layer.weight.grad.cpu(), c["ref_grads"][1], rtol=1e-12, atol=1e-12, msg=c["name"])
            torch.testing.assert_close(layer.bias.grad.cpu(), c["ref_grads"][2], rtol=1e-12, atol=1e-12, msg=c["name"])
        assert gradcheck(layer, args), c["name"]
        n += 1
    assert n == 23


def test_weight_gradients_pass_gradcheck_too():
    """The reference only gradchecks the input; the weight and bias gradients are checked here as well."""
    from spherical_distortion.functional import mapped_convolution, mapped_transposed_convolution
    from spherical_distortion.nn import InterpolationType
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 3, 5, 6, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    w = torch.randn(4, 3, 5, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    b = torch.randn(4, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    m = (torch.rand(4, 5, 5, 2, generator=g, dtype=torch.float64) * torch.tensor([7.0, 6.0]) - 0.5).cuda()
    for it in (InterpolationType.NEAREST, InterpolationType.BILINEAR, InterpolationType.BISPHERICAL):
        assert gradcheck(lambda x_, w_, b_: mapped_convolution(x_, w_, b_, m, 5, it), (x, w, b))
    # transposed: input on the map grid
    xt = torch.randn(2, 4, 4, 5, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    wt = torch.randn(4, 3, 5, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    bt = torch.randn(3, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    assert gradcheck(lambda x_, w_, b_: mapped_transposed_convolution(x_, w_, b_, m, 5, 6, 5, InterpolationType.BILINEAR),
                     (xt, wt, bt))


def test_resample_layer_is_the_adjoint_of_unresample():
    from spherical_distortion.nn import InterpolationType, Resample, Unresample
    g = torch.Generator().manual_seed(6)
    x = torch.randn(2, 3, 8, 10, generator=g, dtype=torch.float64).cuda()
    y = torch.randn(2, 3, 5, 7, generator=g, dtype=torch.float64).cuda()
    m = (torch.rand(5, 7, 2, generator=g, dtype=torch.float64) * torch.tensor([11.0, 9.0]) - 0.5).cuda()
    for it in (InterpolationType.NEAREST, InterpolationType.BILINEAR, InterpolationType.BISPHERICAL):
        lhs = (Unresample(it)(x, m) * y).sum()
        rhs = (x * Resample(it)(y, m, (8, 10))).sum()
        assert abs(lhs - rhs) <= 1e-12 * (abs(lhs) + 1)
    # 3-D inputs get a temporary batch dimension, like the reference's functional wrappers
    assert Unresample()(x[0], m).shape == (3, 5, 7)
