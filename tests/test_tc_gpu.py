"""bf16 tensor-core path (tcgen05) of the mapped convolution family against the CPU oracle.

Tolerance of the tensor-core path (bf16 operands, fp32 accumulation):
    max |got - ref| <= 2e-2 * max |ref|      and      rms(got - ref) <= 5e-3 * rms(ref)
where ref is the float32 oracle on the unrounded inputs."""
import math

import pytest
import torch

from oracle import port

pytestmark = pytest.mark.gpu

MAX_REL, RMS_REL = 2e-2, 5e-3


def _close(got, ref, what):
    d = (got - ref).double()
    mx, rms = d.abs().max().item(), d.pow(2).mean().sqrt().item()
    rmax, rrms = ref.abs().max().item(), ref.double().pow(2).mean().sqrt().item()
    assert mx <= MAX_REL * rmax and rms <= RMS_REL * rrms, \
        "%s: max err %.3e (ref max %.3e), rms err %.3e (ref rms %.3e)" % (what, mx, rmax, rms, rrms)


def _case(seed, B, Cin, Cout, IH, IW, OH, OW, K, interp, P=0, gnomonic=False):
    from sphmap import workloads as wl
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, Cin, IH, IW, generator=g)
    w = wl.kaiming_uniform(g, Cout, Cin, K)
    b = torch.randn(Cout, generator=g) * 0.1
    if gnomonic:
        m = wl.gnomonic_map(IH, IW, IH // OH)
        assert m.shape[:2] == (OH, OW)
    else:
        shape = (OH, OW, K, P, 2) if P else (OH, OW, K, 2)
        m = torch.rand(*shape, generator=g) * torch.tensor([IW + 2.0, IH + 2.0]) - 1.0
    iw = torch.rand(OH, OW, K, P, generator=g) if P else None
    go = torch.randn(B, Cout, OH, OW, generator=g)
    return x, w, b, m, iw, go


CASES = [
    # seed, B, Cin, Cout, IH, IW, OH, OW, K, interp, P, gnomonic
    (1, 2, 64, 128, 32, 64, 32, 64, 9, 1, 0, True),      # encoder layer shape class, stride 1
    (2, 2, 3, 64, 64, 128, 32, 64, 9, 1, 0, True),       # 3 input channels, stride-2 map
    (3, 1, 128, 256, 16, 32, 16, 32, 9, 1, 0, False),    # N = 256, random bilinear map with out-of-range taps
    (4, 2, 16, 32, 24, 40, 17, 23, 5, 2, 0, False),      # bispherical, ragged sizes (tiles with tail pixels)
    (5, 2, 64, 128, 16, 32, 16, 32, 9, 0, 4, False),     # weighted, 4 points, nearest (config-3 class)
    (6, 1, 24, 40, 12, 20, 9, 13, 3, 1, 2, False),       # odd channel counts, weighted bilinear
    (7, 1, 72, 272, 8, 16, 8, 16, 2, 0, 0, False),       # Cout > 256 (two N blocks), Cin padded to 128
    (8, 2, 32, 64, 32, 64, 16, 32, 9, 1, 0, True),       # stride-2 map: the adjoints multiply first on the small grid
    (9, 1, 40, 48, 20, 36, 7, 11, 5, 1, 0, False),       # down-sampling random map, ragged sizes, multiply-first adjoint
    (10, 3, 64, 64, 32, 64, 16, 32, 9, 1, 0, True),      # multiply-first adjoint with 64 input channels (lane-split row gather)
    (11, 1, 128, 32, 21, 37, 7, 11, 5, 1, 0, False),     # the same with two channel groups and ragged destination tiles
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "s%d" % c[0])
def test_conv_forward_and_backward_bf16(case):
    from _gpu_impl import CApi
    seed, B, Cin, Cout, IH, IW, OH, OW, K, interp, P, gn = case
    x, w, b, m, iw, go = _case(seed, B, Cin, Cout, IH, IW, OH, OW, K, interp, P, gn)
    tc = CApi(precision=1)
    out = tc.mapped_conv_forward(x, m, w, b, K, interp, iw)
    _close(out, port.mapped_conv_forward(x, m, w, b, K, interp, iw), "forward")
    gx, gw, gb = tc.mapped_conv_backward(go, m, x, w, b, K, interp, iw)
    rgx, rgw, rgb = port.mapped_conv_backward(go, m, x, w, b, K, interp, iw)
    _close(gx, rgx, "grad_input")
    _close(gw, rgw, "grad_weight")
    _close(gb, rgb, "grad_bias")


@pytest.mark.parametrize("case", CASES[:1] + CASES[3:6] + CASES[7:], ids=lambda c: "s%d" % c[0])
def test_transposed_conv_bf16(case):
    from _gpu_impl import CApi
    seed, B, Cin, Cout, IH, IW, OH, OW, K, interp, P, gn = case
    # transposed: input lives on the (OH, OW) map grid with Cout channels, output on (IH, IW) with Cin channels
    x, w, b, m, iw, go = _case(seed, B, Cin, Cout, IH, IW, OH, OW, K, interp, P, gn)
    g = torch.Generator().manual_seed(seed + 100)
    xt = torch.randn(B, Cout, OH, OW, generator=g)
    bt = torch.randn(Cin, generator=g) * 0.1
    got = torch.randn(B, Cin, IH, IW, generator=g)
    tc = CApi(precision=1)
    out = tc.mapped_transposed_conv_forward(xt, m, w, bt, IH, IW, K, interp, iw)
    _close(out, port.mapped_transposed_conv_forward(xt, m, w, bt, IH, IW, K, interp, iw), "tconv forward")
    gx, gw, gb = tc.mapped_transposed_conv_backward(got, m, xt, w, bt, K, interp, iw)
    rgx, rgw, rgb = port.mapped_transposed_conv_backward(got, m, xt, w, bt, K, interp, iw)
    _close(gx, rgx, "tconv grad_input")
    _close(gw, rgw, "tconv grad_weight")
    _close(gb, rgb, "tconv grad_bias")


def test_bf16_path_is_deterministic():
    from _gpu_impl import CApi
    x, w, b, m, iw, go = _case(11, 2, 64, 128, 32, 64, 32, 64, 9, 1, 0, True)
    tc = CApi(precision=1)
    a = tc.mapped_conv_backward(go, m, x, w, b, 9, 1, None)
    c = tc.mapped_conv_backward(go, m, x, w, b, 9, 1, None)
    for u, v in zip(a, c):
        assert torch.equal(u, v)


# Thin gathered side (channels x K <= 63): one 64-column operand block per tile (forward) and the combined
# dW / dBias / multiply-first dInput kernel (backward).  Shapes outside their cover fall back to the exact kernels.
THIN_CASES = [
    # seed, B, Cin, Cout, IH, IW, OH, OW, K, interp, P, gnomonic
    (21, 3, 3, 64, 64, 128, 32, 64, 9, 1, 0, True),      # RGB first layer, stride-2 gnomonic map
    (22, 2, 1, 16, 20, 24, 10, 12, 4, 0, 0, False),      # one channel, nearest, 120 pixels: a partial last step
    (23, 2, 4, 32, 18, 40, 9, 16, 9, 2, 0, False),       # bispherical
    (24, 1, 2, 48, 16, 32, 16, 32, 5, 1, 2, False),      # weighted bilinear, two points per slot
    (25, 2, 3, 64, 30, 50, 15, 25, 9, 1, 0, False),      # width not a multiple of 4, 375 pixels: the exact kernels
    (26, 2, 3, 128, 32, 64, 16, 32, 9, 1, 0, True),      # forward thin (N = 128), backward on the exact kernels
    (27, 5, 3, 64, 16, 32, 8, 16, 7, 1, 0, False),       # five images (a partial image group in the plan gather)
    (28, 1, 1, 16, 12, 16, 6, 8, 63, 1, 0, False),       # 63 columns: the ones column of the backward is the last one
    (29, 2, 7, 32, 12, 16, 6, 8, 9, 0, 0, False),        # seven channels: forward thin (general gather), backward exact
    (30, 9, 2, 64, 16, 16, 16, 16, 3, 1, 0, False),      # nine images: two image groups of the plan gather, K odd
]


@pytest.mark.parametrize("case", THIN_CASES, ids=lambda c: "s%d" % c[0])
def test_thin_layer_bf16(case):
    from sphmap import capi
    seed, B, Cin, Cout, IH, IW, OH, OW, K, interp, P, gn = case
    x, w, b, m, iw, go = _case(seed, B, Cin, Cout, IH, IW, OH, OW, K, interp, P, gn)
    ref = port.mapped_conv_forward(x, m, w, b, K, interp, iw)
    rgx, rgw, rgb = port.mapped_conv_backward(go * (ref > 0), m, x, w, b, K, interp, iw)
    d = lambda t: None if t is None else t.cuda()
    xd, wd, bd, md, iwd, god = d(x), d(w), d(b), d(m), d(iw), d(go)
    # forward with the fused ReLU and the channels-last copy of the output
    cl = capi.companion(B, Cout, OH, OW, "cuda") if Cout % 8 == 0 else None
    try:
        out = capi.conv_forward_cl(xd, None, md, wd, bd, K, interp, iwd, capi.BF16, True, out_cl=cl)
    except capi.Unsupported:
        cl = None
        out = capi.conv_forward_cl(xd, None, md, wd, bd, K, interp, iwd, capi.BF16, True, out_cl=None)
    _close(out.cpu(), ref.clamp(min=0), "forward + relu")
    if cl is not None:
        import ctypes
        cp = int(capi.lib.sph_conv_companion_channels(ctypes.c_int64(Cout)))
        v = cl[:B * (OH * OW + 1) * cp * 2].view(torch.bfloat16).view(B, OH * OW + 1, cp)
        assert torch.equal(v[:, :OH * OW, :Cout].float(), out.to(torch.bfloat16).float().flatten(2).transpose(1, 2))
        assert (v[:, OH * OW] == 0).all() and (v[:, :, Cout:] == 0).all()
    # backward: the combined call where it applies, and the separate entry points (same kernels, same results)
    act = (ref > 0).float().cuda()     # the oracle's activation pattern, so that the masks agree
    plan = capi.plan_build(md, iwd, OH * OW, K, interp, IH, IW)
    gx = capi.conv_relu_backward_input(god, act, plan, wd, IH, IW, K, capi.BF16)
    gw, gb = capi.conv_relu_backward_weight(god, act, xd, md, K, interp, iwd, capi.BF16)
    _close(gx.cpu(), rgx, "grad_input")
    _close(gw.cpu(), rgw, "grad_weight")
    _close(gb.cpu(), rgb, "grad_bias")
    try:
        cx, cw, cb = capi.conv_backward_cl(god, act, xd, None, plan, md, wd, K, interp, iwd, capi.BF16)
    except capi.Unsupported:
        assert Cout > 64 or (OH * OW) % 8 != 0 or Cin > 4
    else:
        assert torch.equal(cx, gx) and torch.equal(cw, gw) and torch.equal(cb, gb)
        cx2, cw2, cb2 = capi.conv_backward_cl(god, act, xd, None, plan, md, wd, K, interp, iwd, capi.BF16)
        assert torch.equal(cx, cx2) and torch.equal(cw, cw2) and torch.equal(cb, cb2)   # run-to-run identical
