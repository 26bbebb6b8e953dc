"""The BASELINE configurations on the GPU: oracle comparisons at sizes the CPU oracle finishes in seconds, and
size-independent properties (adjointness, linearity, index consistency) at the configurations' full sizes."""
import pytest
import torch

from oracle import port

pytestmark = pytest.mark.gpu


def _capi():
    from sphmap import capi
    return capi


def _rel(a, b):
    return ((a - b).double().norm() / b.double().norm().clamp_min(1e-30)).item()


def test_config0_forward_full_size_exact_and_bf16():
    """Config 0 (B=2, 16->32, 64x128, bilinear 3x3 gnomonic map): the reference's CPU-runnable case, at full size."""
    from sphmap import workloads as wl
    c, capi = wl.config0(), _capi()
    ref = port.mapped_conv_forward(c["x"], c["map"], c["weight"], c["bias"], 9, 1)
    d = {k: v.cuda() for k, v in c.items() if torch.is_tensor(v)}
    got = capi.conv_forward(d["x"], d["map"], d["weight"], d["bias"], 9, 1).cpu()
    torch.testing.assert_close(got, ref, rtol=1e-5, atol=1e-5 * ref.abs().max().item())
    tc = capi.conv_forward(d["x"], d["map"], d["weight"], d["bias"], 9, 1, None, capi.BF16).cpu()
    assert (tc - ref).abs().max() <= 2e-2 * ref.abs().max() and _rel(tc, ref) <= 5e-3


def test_config1_resampling_full_size():
    """Config 1: gather bit exact against the oracle, scatter and the normalised scatter within 1e-5."""
    from sphmap import workloads as wl
    c, capi = wl.config1(), _capi()
    x, m = c["x"], c["map"]
    H, W = c["out_hw"]
    xd, md = x.cuda(), m.cuda()
    y = capi.resample_from_map(xd, md, 1)
    assert torch.equal(y.cpu(), port.resample_from_map(x, m, 1))
    plan = capi.plan_build(md, None, m.shape[0] * m.shape[1], 1, 1, H, W)
    back = capi.resample_to_map(y, plan, H, W)
    ref_back = port.resample_to_map(y.cpu(), m, H, W, 1)
    torch.testing.assert_close(back.cpu(), ref_back, rtol=1e-5, atol=1e-6)
    # normalisation as in the reference's sphere_ops: scatter(y) / (scatter(1) + 1e-12); the denominator depends on the map only
    ones = torch.ones(1, 1, m.shape[0], m.shape[1], device="cuda")
    wsum = capi.resample_to_map(ones, plan, H, W)
    norm = back / (wsum + 1e-12)
    ref_norm = ref_back / (port.resample_to_map(ones.cpu(), m, H, W, 1) + 1e-12)
    torch.testing.assert_close(norm.cpu(), ref_norm, rtol=1e-5, atol=1e-6)
    # adjointness of gather and scatter at full size: <gather(x), y> == <x, scatter(y)>
    lhs = (y.double() * y.double()).sum()
    rhs = (xd.double() * back.double()).sum()
    assert abs(lhs - rhs) / abs(lhs) < 1e-6


def test_config2_pooling_full_size_bit_exact():
    """Config 2 at full size (B=8, C=64, 256x512 -> 128x256, K=9, nearest, random map): values and indices bit
    exact against the oracle run with the CUDA build's sentinel; backward within 1e-5; index consistency."""
    from sphmap import workloads as wl
    c, capi = wl.config2(), _capi()
    x, m, go = c["x"], c["map"], c["grad_output"]
    xd, md, god = x.cuda(), m.cuda(), go.cuda()
    out, idx = capi.mapped_max_pool(xd, md, 9, 0)
    rout, ridx = port.mapped_max_pool(x, m, 9, 0, cuda_sentinel=True)
    assert torch.equal(out.cpu(), rout) and torch.equal(idx.cpu(), ridx)
    # where the reference's CPU build has an index (>= 0) it is the same index and value
    cout, cidx = port.mapped_max_pool(x, m, 9, 0)
    keep = cidx >= 0
    assert torch.equal(out.cpu()[keep], cout[keep]) and torch.equal(idx.cpu()[keep], cidx[keep])
    gin = capi.mapped_max_unpool(god, idx, md, x.shape[2], x.shape[3], 9, 0)
    rgin = port.mapped_max_unpool(go, ridx, m, x.shape[2], x.shape[3], 9, 0)
    torch.testing.assert_close(gin.cpu(), rgin, rtol=1e-5, atol=1e-5)
    # every index names a slot of its own output position: idx - o * 2K is an even number in [0, 2K)
    o = torch.arange(out.shape[2] * out.shape[3], device="cuda").view(1, 1, out.shape[2], out.shape[3])
    r = idx - o * 18
    assert ((r >= 0) & (r < 18) & (r % 2 == 0)).all()
    # gradient mass is conserved by the argmax backward (every tap of a random in-range nearest map is valid)
    assert abs(gin.double().sum() - god.double().sum()) < 1e-3 * god.double().abs().sum()


@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_config3_weighted_conv_reduced_size_against_oracle(precision):
    """Config 3's operators (weighted 4-point nearest conv fwd/bwd and the transposed conv) at 1/64 of the pixels."""
    from sphmap import workloads as wl
    from _gpu_impl import CApi
    c = wl.config3(B=1, H=32, W=64)
    impl = CApi(precision=1 if precision == "bf16" else 0)

    def close(a, r):
        if precision == "bf16":
            assert (a - r).abs().max() <= 2e-2 * r.abs().max() and _rel(a, r) <= 5e-3
        else:
            torch.testing.assert_close(a, r, rtol=1e-5, atol=1e-5 * r.abs().max().item())

    close(impl.mapped_conv_forward(c["x"], c["map"], c["weight"], c["bias"], 9, 0, c["iw"]),
          port.mapped_conv_forward(c["x"], c["map"], c["weight"], c["bias"], 9, 0, c["iw"]))
    for a, r in zip(impl.mapped_conv_backward(c["grad_output"], c["map"], c["x"], c["weight"], c["bias"], 9, 0, c["iw"]),
                    port.mapped_conv_backward(c["grad_output"], c["map"], c["x"], c["weight"], c["bias"], 9, 0, c["iw"])):
        close(a, r)
    t = c["t"]
    close(impl.mapped_transposed_conv_forward(t["x"], t["map"], t["weight"], t["bias"], t["oh"], t["ow"], 9, 0, t["iw"]),
          port.mapped_transposed_conv_forward(t["x"], t["map"], t["weight"], t["bias"], t["oh"], t["ow"], 9, 0, t["iw"]))
    for a, r in zip(impl.mapped_transposed_conv_backward(t["grad_output"], t["map"], t["x"], t["weight"], t["bias"], 9, 0, t["iw"]),
                    port.mapped_transposed_conv_backward(t["grad_output"], t["map"], t["x"], t["weight"], t["bias"], 9, 0, t["iw"])):
        close(a, r)


@pytest.mark.parametrize("precision,tol", [("fp32", 1e-4), ("bf16", 1e-2)])
def test_config3_full_size_adjointness(precision, tol):
    """Config 3 at full size (B=16, 64->128, 256x512, K=9, P=4): the backward operators are the adjoints of the
    forward one: <conv(x), g> = <x, dX(g)> = <W, dW(g)> (+ <bias, dB>), which needs no oracle."""
    from sphmap import workloads as wl
    capi = _capi()
    c = wl.config3()
    prec = capi.BF16 if precision == "bf16" else capi.EXACT
    x, w, m, iw, g = (c[k].cuda() for k in ("x", "weight", "map", "iw", "grad_output"))
    zero_bias = torch.zeros(128, device="cuda")
    H, W = x.shape[2], x.shape[3]
    out = capi.conv_forward(x, m, w, zero_bias, 9, 0, iw, prec)
    lhs = (out.double() * g.double()).sum().item()
    plan = capi.plan_build(m, iw, H * W, 9, 0, H, W)
    gx = capi.conv_backward_input(g, plan, w, H, W, 9, prec)
    gw, gb = capi.conv_backward_weight(g, x, m, 9, 0, iw, prec)
    scale = out.double().norm().item() * g.double().norm().item()
    assert abs(lhs - (x.double() * gx.double()).sum().item()) <= tol * scale
    assert abs(lhs - (w.double() * gw.double()).sum().item()) <= tol * scale
    torch.testing.assert_close(gb, g.sum((0, 2, 3)), rtol=1e-4, atol=1e-2)
    # linearity in the input at full size
    out2 = capi.conv_forward(2.0 * x, m, w, zero_bias, 9, 0, iw, prec)
    assert _rel(out2, 2.0 * out) <= (1e-6 if precision == "fp32" else 1e-2)


@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_config4_encoder_stack_small_resolution(precision):
    """The four-layer encoder (config 4) at 32x64 input, batch 2: every layer's output and gradients against the oracle."""
    from sphmap import capi, workloads as wl
    from sphmap.parallel import EncoderStack
    cfg = wl.config4(B=2, H=32, W=64)
    dev = torch.device("cuda:0")
    stack = EncoderStack(cfg, dev, capi.BF16 if precision == "bf16" else capi.EXACT, 2)
    stack.step(cfg["x"].to(dev), cfg["grad_output"].to(dev))
    # oracle: same forward / backward on the CPU
    acts, ins, h = [], [], cfg["x"]
    for li in range(4):
        ins.append(h)
        h = port.mapped_conv_forward(h, cfg["maps"][li], cfg["weights"][li], cfg["biases"][li], 9, 1).relu_()
        acts.append(h)
    g = cfg["grad_output"]
    for li in reversed(range(4)):
        g = g * (acts[li] > 0)
        gx, gw, gb = port.mapped_conv_backward(g, cfg["maps"][li], ins[li], cfg["weights"][li], cfg["biases"][li], 9, 1)
        if precision == "fp32":
            for name, a, r in (("gw", stack.gw[li], gw), ("gb", stack.gb[li], gb), ("gx", stack.gx[li], gx)):
                assert _rel(a.cpu(), r) <= 1e-4, (name, li)
        else:
            # Through a chain of ReLUs the bf16 forward flips the sign of a few near-zero activations, which moves
            # whole gradient entries in or out of the mask; the per-operator tolerance is checked in test_tc_gpu.py,
            # here the gradients of the whole chain must still point the same way.
            for name, a, r in (("gw", stack.gw[li], gw), ("gb", stack.gb[li], gb), ("gx", stack.gx[li], gx)):
                cos = torch.nn.functional.cosine_similarity(a.cpu().flatten().double(), r.flatten().double(), dim=0).item()
                assert cos >= 0.99, (name, li, cos)
        g = gx
    assert _rel(stack.acts[3].cpu(), acts[3]) <= (1e-2 if precision == "bf16" else 1e-5)
