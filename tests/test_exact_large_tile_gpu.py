"""The large-tile kernels of the exact float32 path (128 / 64 x 128 gather-GEMM, 128 x 128 weight gradient, the
multiply-first adjoint) on shapes that do not fill their tiles and fast paths: odd channel counts, ragged images, every
interpolation type, weighted maps, down-sampling maps.  Against the CPU oracle at the exact path's tolerance
|err| <= 1e-5 |ref| + 1e-5 max|ref|."""
import pytest
import torch

from oracle import port

pytestmark = pytest.mark.gpu

CASES = [
    # seed, B, Cin, Cout, IH, IW, OH, OW, K, interp, P
    (1, 2, 40, 72, 21, 37, 13, 22, 5, 1, 0),      # odd channel counts (no eight-channel fast path everywhere), ragged sizes
    (2, 1, 64, 128, 16, 32, 16, 32, 9, 0, 0),     # nearest, full tiles
    (3, 2, 72, 56, 12, 20, 12, 20, 3, 2, 0),      # bispherical, 56 output rows (64-row tile), 72 gathered channels
    (4, 1, 64, 96, 14, 18, 14, 18, 4, 1, 2),      # weighted bilinear (weight gradient on the general kernel)
    (5, 2, 128, 64, 16, 24, 16, 24, 4, 0, 3),     # weighted nearest, three points (weight-gradient tile for weighted nearest maps)
    (6, 2, 56, 24, 20, 36, 7, 11, 5, 1, 0),       # down-sampling map: the adjoints multiply first (K * Cin = 120 rows)
    (7, 3, 48, 64, 32, 64, 16, 32, 9, 1, 0),      # stride-2 gnomonic-like size ratio, 64 rows: multiply-first with 64-row tiles
]


def _close(got, ref, what):
    torch.testing.assert_close(got.cpu(), ref, rtol=1e-5, atol=1e-5 * max(1.0, float(ref.abs().max())), msg=what)


@pytest.mark.parametrize("case", CASES, ids=lambda c: "s%d" % c[0])
def test_exact_conv_and_transposed_conv(case):
    from _gpu_impl import CApi
    seed, B, Cin, Cout, IH, IW, OH, OW, K, interp, P = case
    g = torch.Generator().manual_seed(1000 + seed)
    x = torch.randn(B, Cin, IH, IW, generator=g)
    w = torch.randn(Cout, Cin, K, generator=g) / (Cin * K) ** 0.5
    b = torch.randn(Cout, generator=g) * 0.1
    shape = (OH, OW, K, P, 2) if P else (OH, OW, K, 2)
    m = torch.rand(*shape, generator=g) * torch.tensor([IW + 2.0, IH + 2.0]) - 1.0
    iw = torch.rand(OH, OW, K, P, generator=g) if P else None
    go = torch.randn(B, Cout, OH, OW, generator=g)
    impl = CApi()          # exact precision
    _close(impl.mapped_conv_forward(x, m, w, b, K, interp, iw), port.mapped_conv_forward(x, m, w, b, K, interp, iw), "forward")
    for name, a, r in zip(("grad_input", "grad_weight", "grad_bias"), impl.mapped_conv_backward(go, m, x, w, b, K, interp, iw),
                          port.mapped_conv_backward(go, m, x, w, b, K, interp, iw)):
        _close(a, r, name)
    # transposed: input on the (OH, OW) map grid with Cout channels, output on (IH, IW) with Cin channels
    xt = torch.randn(B, Cout, OH, OW, generator=g)
    wt = torch.randn(Cout, Cin, K, generator=g) / (Cout * K) ** 0.5
    bt = torch.randn(Cin, generator=g) * 0.1
    got = torch.randn(B, Cin, IH, IW, generator=g)
    _close(impl.mapped_transposed_conv_forward(xt, m, wt, bt, IH, IW, K, interp, iw),
           port.mapped_transposed_conv_forward(xt, m, wt, bt, IH, IW, K, interp, iw), "tconv forward")
    for name, a, r in zip(("tconv grad_input", "tconv grad_weight", "tconv grad_bias"),
                          impl.mapped_transposed_conv_backward(got, m, xt, wt, bt, K, interp, iw),
                          port.mapped_transposed_conv_backward(got, m, xt, wt, bt, K, interp, iw)):
        _close(a, r, name)
