"""Pins the plain-C oracle (oracle/sph_oracle.c): it must reproduce the
known-answer vectors of the reference's own test suite and the outputs of the
reference's compiled CPU modules stored in tests/golden/ (CPU only)."""
import os

import pytest
import torch

from oracle import port, ref


def _load(golden_dir, name):
    return torch.load(os.path.join(golden_dir, name), weights_only=False)


def _run(c, impl):
    """Evaluate one fixture case with `impl` (oracle.port or oracle.ref); returns (output, idx, grads)."""
    x, m, iw, it, K = c["input"], c["sample_map"], c.get("interp_weights"), c["interp"], c.get("kernel_size")
    op = c["op"]
    if op == "conv":
        out = impl.mapped_conv_forward(x, m, c["weight"], c["bias"], K, it, iw)
        go = c.get("grad_output", torch.ones_like(out))
        return out, None, list(impl.mapped_conv_backward(go, m, x, c["weight"], c["bias"], K, it, iw))
    if op == "tconv":
        out = impl.mapped_transposed_conv_forward(x, m, c["weight"], c["bias"], c["oh"], c["ow"], K, it, iw)
        go = c.get("grad_output", torch.ones_like(out))
        return out, None, list(impl.mapped_transposed_conv_backward(go, m, x, c["weight"], c["bias"], K, it, iw))
    if op == "pool":
        out, idx = impl.mapped_max_pool(x, m, K, it, iw)
        go = c.get("grad_output", torch.ones_like(out))
        return out, idx, [impl.mapped_max_unpool(go, idx, m, x.shape[2], x.shape[3], K, it, iw)]
    if op == "resample":
        out = impl.resample_from_map(x, m, it, iw)
        go = c.get("grad_output", torch.ones_like(out))
        return out, None, [impl.resample_to_map(go, m, x.shape[2], x.shape[3], it, iw)]
    raise ValueError(op)


def _tol(dtype):
    return dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=1e-12, atol=1e-13)


def test_port_reproduces_reference_known_answers(golden_dir):
    kats = _load(golden_dir, "reference_kats.pt")
    assert len(kats) == 23
    for c in kats:
        out, idx, grads = _run(c, port)
        exp = c["expected"].to(out.dtype).expand_as(out)
        torch.testing.assert_close(out, exp, rtol=1e-7, atol=1e-9, msg=c["name"])
        torch.testing.assert_close(out, c["ref_output"], **_tol(out.dtype), msg=c["name"])
        if idx is not None:
            assert torch.equal(idx, c["ref_idx"]), c["name"]
        for a, b in zip(grads, c["ref_grads"]):
            torch.testing.assert_close(a, b, **_tol(a.dtype), msg=c["name"])


def test_port_matches_reference_on_random_cases(golden_dir):
    cases = _load(golden_dir, "reference_random.pt")
    n = 0
    for c in cases:
        if c["op"] == "pool_sentinel":
            continue
        out, idx, grads = _run(c, port)
        if c["op"] in ("pool", "resample"):
            assert torch.equal(out, c["ref_output"]), (c["op"], c["seed"], c["interp"])  # gathers are bit exact
        else:
            torch.testing.assert_close(out, c["ref_output"], **_tol(out.dtype))
        if idx is not None:
            assert torch.equal(idx, c["ref_idx"])
        for a, b in zip(grads, c["ref_grads"]):
            torch.testing.assert_close(a, b, **_tol(a.dtype))
        n += 1
    assert n == 48


def test_port_max_pool_sentinels(golden_dir):
    """CPU build of the reference: smallest positive normal + idx -1; CUDA build: -FLT_MAX."""
    c = [c for c in _load(golden_dir, "reference_random.pt") if c["op"] == "pool_sentinel"][0]
    out, idx = port.mapped_max_pool(c["input"], c["sample_map"], c["kernel_size"], c["interp"])
    assert torch.equal(out, c["ref_output"]) and torch.equal(idx, c["ref_idx"])
    assert (idx < 0).any(), "fixture must exercise the sentinel"
    out2, idx2 = port.mapped_max_pool(c["input"], c["sample_map"], c["kernel_size"], c["interp"], cuda_sentinel=True)
    keep = idx >= 0
    assert torch.equal(out2[keep], out[keep]) and torch.equal(idx2[keep], idx[keep])
    assert (idx2 >= 0).all()


def test_nearest_rounds_half_away_from_zero():
    x = torch.arange(12, dtype=torch.float64).view(1, 1, 3, 4)
    m = torch.tensor([[[0.5, 0.0], [1.5, 0.0], [2.5, 0.0], [-0.5, 0.0], [3.5, 0.0], [0.0, 1.5]]], dtype=torch.float64)
    y = port.resample_from_map(x, m, 0)
    assert y.flatten().tolist() == [1.0, 2.0, 3.0, 0.0, 0.0, 8.0]


@pytest.mark.skipif(not ref.available(), reason="compiled reference modules not present")
def test_port_matches_live_reference_float32_config0_shape():
    """Config-0 shape (B=2, 16->32, 64x128, K=9, bilinear, fp32) against the live reference."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 16, 64, 128, generator=g)
    m = torch.rand(64, 128, 9, 2, generator=g) * torch.tensor([130.0, 66.0]) - 1.0
    w = torch.randn(32, 16, 9, generator=g) / 12
    b = torch.randn(32, generator=g) * 0.01
    a = port.mapped_conv_forward(x, m, w, b, 9, 1)
    r = ref.mapped_conv_forward(x, m, w, b, 9, 1)
    torch.testing.assert_close(a, r, rtol=1e-5, atol=1e-5)


def _run_sibling(c, impl):
    if c["op"] == "avgpool":
        x, m, iw, it, K = c["input"], c["sample_map"], c["interp_weights"], c["interp"], c["kernel_size"]
        return impl.mapped_avg_pool(x, m, K, it, iw), [impl.mapped_avg_unpool(c["grad_output"], m, x.shape[2], x.shape[3], K, it, iw)]
    if c["op"] == "uv":
        tex = c["input"]
        return (impl.resample_from_uv_maps(tex, c["quad_idx"], c["tex_uv"], c["interp"]),
                [impl.resample_to_uv_maps(c["grad_output"], c["quad_idx"], c["tex_uv"], *tex.shape[2:], c["interp"])])
    if c["op"] == "voting":
        return impl.voting_resample_to_map(c["input"], c["sample_map"], c["oh"], c["ow"], c["num_candidates"]), []
    raise ValueError(c["op"])


def test_port_matches_reference_on_sibling_operators(golden_dir):
    """Average pooling, UV-map and voting resampling of the plain-C oracle against the compiled reference's outputs."""
    n = 0
    for c in _load(golden_dir, "reference_siblings.pt"):
        if c["op"] == "map":
            continue
        out, grads = _run_sibling(c, port)
        if c["op"] == "voting":
            assert torch.equal(out, c["ref_output"]), c["seed"]
        else:
            # gathers add K values in the reference's order: bit exact; the scatters add in any order there
            assert torch.equal(out, c["ref_output"]), (c["op"], c["seed"], c["interp"])
            for a, b in zip(grads, c["ref_grads"]):
                torch.testing.assert_close(a, b, **_tol(a.dtype))
        n += 1
    assert n == 21


def test_workload_gnomonic_map_matches_reference_builder(golden_dir):
    """The benchmark's own map generator (sphmap.workloads.gnomonic_map) against the reference's Python builder."""
    from sphmap import workloads as wl
    for c in _load(golden_dir, "reference_siblings.pt"):
        if c["op"] == "map" and c["kind"] == "inverse_gnomonic" and c["kh"] == c["kw"] and c["dilation"] == 1:
            got = wl.gnomonic_map(c["H"], c["W"], c["stride"], c["kh"], dtype=torch.float64)
            ok = ~torch.isnan(c["f64"])   # even kernels: the reference's zero differential evaluates to 0/0
            torch.testing.assert_close(got[ok], c["f64"][ok], rtol=0, atol=1e-9)
