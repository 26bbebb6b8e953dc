"""bf16 tensor-core path (tcgen05) of the mapped convolution family against the CPU oracle.

Tolerance of the tensor-core path (bf16 operands, fp32 accumulation), stated per BASELINE.json:
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
