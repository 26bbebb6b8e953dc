"""Parity of the CUDA library with the reference on the committed golden
fixtures: the reference test suite's known-answer vectors and the seeded
random cases evaluated with the reference's compiled CPU modules.

Bars: gathers (resample_from_map, pooled values) and argmax indices bit exact;
everything else within rtol 1e-5 (float32) / 1e-12 (float64), the tolerance
of the exact path."""
import os

import pytest
import torch

from test_oracle import _load, _run, _tol as _strict_tol

pytestmark = pytest.mark.gpu


def _close(a, b, msg):
    """|a - b| <= rtol * |b| + atol with atol tied to the tensor's scale: sums of many float32 products carry a
    rounding error proportional to the magnitude of the terms, not of the (possibly cancelling) result, and the
    GPU kernels add their partial sums in a different order than the reference's SGEMM."""
    tol = _strict_tol(a.dtype)
    scale = float(b.abs().max()) if b.numel() else 0.0
    torch.testing.assert_close(a, b, rtol=tol["rtol"], atol=max(tol["atol"], tol["rtol"] * scale), msg=msg)


@pytest.fixture(scope="module", params=["capi", "plugin"])
def impl(request):
    from _gpu_impl import CApi, Plugin
    return CApi() if request.param == "capi" else Plugin()


def test_reference_known_answers(impl, golden_dir):
    for c in _load(golden_dir, "reference_kats.pt"):
        out, idx, grads = _run(c, impl)
        exp = c["expected"].to(out.dtype).expand_as(out)
        torch.testing.assert_close(out, exp, rtol=1e-7, atol=1e-9, msg=c["name"])
        if c["op"] in ("pool", "resample"):
            assert torch.equal(out, c["ref_output"]), c["name"]
        else:
            _close(out, c["ref_output"], c["name"])
        if idx is not None:
            assert torch.equal(idx, c["ref_idx"]), c["name"]
        for a, b in zip(grads, c["ref_grads"]):
            _close(a, b, c["name"])


def test_reference_random_cases(impl, golden_dir):
    n = 0
    for c in _load(golden_dir, "reference_random.pt"):
        if c["op"] == "pool_sentinel":
            continue
        tag = (c["op"], c["seed"], c["interp"], str(c["input"].dtype), c.get("interp_weights") is not None)
        out, idx, grads = _run(c, impl)
        if c["op"] in ("pool", "resample"):
            assert torch.equal(out, c["ref_output"]), tag
        else:
            _close(out, c["ref_output"], str(tag))
        if idx is not None:
            assert torch.equal(idx, c["ref_idx"]), tag
        for a, b in zip(grads, c["ref_grads"]):
            _close(a, b, str(tag))
        n += 1
    assert n == 48


def test_max_pool_sentinel_is_the_cuda_build_one(impl, golden_dir):
    """Where the reference CPU build returns idx -1 (nothing above its positive sentinel) the CUDA
    semantics (-FLT_MAX start) still pick the true maximum; elsewhere both agree bit for bit."""
    from oracle import port
    c = [c for c in _load(golden_dir, "reference_random.pt") if c["op"] == "pool_sentinel"][0]
    out, idx = impl.mapped_max_pool(c["input"], c["sample_map"], c["kernel_size"], c["interp"])
    keep = c["ref_idx"] >= 0
    assert torch.equal(out[keep], c["ref_output"][keep]) and torch.equal(idx[keep], c["ref_idx"][keep])
    o2, i2 = port.mapped_max_pool(c["input"], c["sample_map"], c["kernel_size"], c["interp"], cuda_sentinel=True)
    assert torch.equal(out, o2) and torch.equal(idx, i2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("interp,P", [(0, 0), (1, 0), (2, 3), (1, 2)])
def test_exact_path_with_wide_channels(impl, dtype, interp, P):
    """Channel counts beyond the thin-contraction kernels (Cin*K > 32): the tiled exact SIMT kernels, conv and
    transposed conv, against the CPU oracle on seeded inputs (ragged sizes, out-of-range coordinates)."""
    from oracle import port
    g = torch.Generator().manual_seed(4000 + 10 * interp + P)
    B, Cin, Cout, IH, IW, OH, OW, K = 2, 12, 70, 9, 13, 7, 11, 5
    x = torch.randn(B, Cin, IH, IW, generator=g, dtype=dtype)
    shape = (OH, OW, K, P, 2) if P else (OH, OW, K, 2)
    m = (torch.rand(*shape, generator=g, dtype=torch.float64) * torch.tensor([IW + 3.0, IH + 3.0]) - 1.5).to(dtype)
    iw = torch.rand(OH, OW, K, P, generator=g, dtype=dtype) if P else None
    w = torch.randn(Cout, Cin, K, generator=g, dtype=dtype) / 8
    b = torch.randn(Cout, generator=g, dtype=dtype)
    go = torch.randn(B, Cout, OH, OW, generator=g, dtype=dtype)
    def close(a, r):
        # 1e-5 (fp32) / 1e-12 (fp64) relative to the tensor's scale: sums of 60 to ~10^4 terms differ from the
        # oracle only by summation order
        rt = 1e-5 if dtype == torch.float32 else 1e-12
        torch.testing.assert_close(a, r, rtol=rt, atol=rt * float(r.abs().max()))

    close(impl.mapped_conv_forward(x, m, w, b, K, interp, iw), port.mapped_conv_forward(x, m, w, b, K, interp, iw))
    for a, r in zip(impl.mapped_conv_backward(go, m, x, w, b, K, interp, iw),
                    port.mapped_conv_backward(go, m, x, w, b, K, interp, iw)):
        close(a, r)
    # transposed: input on the map grid with Cout channels, output on (IH, IW) with Cin channels
    xt = torch.randn(B, Cout, OH, OW, generator=g, dtype=dtype)
    bt = torch.randn(Cin, generator=g, dtype=dtype)
    got = torch.randn(B, Cin, IH, IW, generator=g, dtype=dtype)
    close(impl.mapped_transposed_conv_forward(xt, m, w, bt, IH, IW, K, interp, iw),
          port.mapped_transposed_conv_forward(xt, m, w, bt, IH, IW, K, interp, iw))
    for a, r in zip(impl.mapped_transposed_conv_backward(got, m, xt, w, bt, K, interp, iw),
                    port.mapped_transposed_conv_backward(got, m, xt, w, bt, K, interp, iw)):
        close(a, r)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_resample_to_map_many_planes(dtype):
    """Enough (batch, channel) planes to select the four-pixels-per-thread scatter kernel; same bar as the rest."""
    from _gpu_impl import CApi
    from oracle import port
    g = torch.Generator().manual_seed(77)
    x = torch.randn(8, 80, 20, 30, generator=g, dtype=dtype)
    m = (torch.rand(20, 30, 2, generator=g, dtype=torch.float64) * torch.tensor([130.0, 66.0]) - 1.0).to(dtype)
    got = CApi().resample_to_map(x, m, 64, 128, 1)
    ref = port.resample_to_map(x, m, 64, 128, 1)
    rt = 1e-5 if dtype == torch.float32 else 1e-12
    torch.testing.assert_close(got, ref, rtol=rt, atol=rt)
    assert torch.equal(got, CApi().resample_to_map(x, m, 64, 128, 1))      # deterministic
