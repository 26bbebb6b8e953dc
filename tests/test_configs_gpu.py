"""The five benchmark configurations on the GPU, at the sizes the benchmark times them.

Every operator is compared with the CPU oracle (the reference's own compiled CPU modules when they were built,
else the plain-C restatement) on the same seeded tensors, plus size-independent properties (adjointness, linearity,
index consistency).  Tolerances, stated once:

    exact path (float32 arithmetic)   |got - ref| <= 1e-5 * |ref| + 1e-5 * max|ref|   element-wise
                                      (the absolute floor follows the tensor's scale because the kernels add the
                                      partial sums of the contraction in another order than the reference's SGEMM)
    bf16 tensor-core path             max|got - ref| <= 2e-2 * max|ref|   and   rms(got - ref) <= 5e-3 * rms(ref)

Gathers, pooled values and indices are compared bit for bit."""
import pytest
import torch

from oracle import port, ref

pytestmark = pytest.mark.gpu

MAX_REL, RMS_REL = 2e-2, 5e-3


def _oracle():
    """The compiled reference modules when present (they use the host's BLAS for the contraction, which is what makes
    full-size images affordable), else the plain-C port."""
    return ref if ref.available() else port


def _close(got, want, precision, what):
    got, want = got.detach().cpu(), want.detach().cpu()
    d = (got - want).double()
    mx, rms = d.abs().max().item(), d.pow(2).mean().sqrt().item()
    rmax, rrms = want.abs().max().item(), want.double().pow(2).mean().sqrt().item()
    if precision == "bf16":
        assert mx <= MAX_REL * rmax and rms <= RMS_REL * rrms, \
            "%s: max err %.3e (ref max %.3e), rms err %.3e (ref rms %.3e)" % (what, mx, rmax, rms, rrms)
    else:
        bad = d.abs() > 1e-5 * want.abs().double() + 1e-5 * rmax
        assert not bad.any(), "%s: %d elements off, max err %.3e (ref max %.3e), rms err %.3e (ref rms %.3e)" % (
            what, int(bad.sum()), mx, rmax, rms, rrms)


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




def _encoder_oracle_chain(cfg):
    """Forward and backward of the four-layer stack on the CPU oracle: per layer its input, its pre-activation output,
    its rectified output, the gradient w.r.t. the rectified output, the masked gradient and the three gradients."""
    o = _oracle()
    L, h = [], cfg["x"]
    for li in range(4):
        pre = o.mapped_conv_forward(h, cfg["maps"][li], cfg["weights"][li], cfg["biases"][li], 9, 1)
        act = pre.clamp_min(0)
        L.append(dict(x=h, pre=pre, act=act))
        h = act
    g = cfg["grad_output"]
    for li in reversed(range(4)):
        L[li]["g"] = g
        L[li]["gm"] = g * (L[li]["act"] > 0)
        gx, gw, gb = o.mapped_conv_backward(L[li]["gm"], cfg["maps"][li], L[li]["x"], cfg["weights"][li], cfg["biases"][li], 9, 1)
        L[li].update(gx=gx, gw=gw, gb=gb)
        g = gx
    return L


def _check_encoder_per_operator(cfg, precision, layers=(0, 1, 2, 3)):
    """Every operator of every layer on the GPU, fed the oracle's own (exact) activations and masked gradients so that
    one layer's rounding cannot flip a ReLU of the next: plain forward / dInput / dW / dBias, and the fused-ReLU entry
    points the benchmark times (they get the unmasked gradient and the rectified output)."""
    from sphmap import capi
    prec = capi.BF16 if precision == "bf16" else capi.EXACT
    L = _encoder_oracle_chain(cfg)
    for li in layers:
        ci, co, (ih, iw), (oh, ow), s = cfg["layers"][li]
        r = L[li]
        m, w, b = cfg["maps"][li].cuda(), cfg["weights"][li].cuda(), cfg["biases"][li].cuda()
        x, gm, g, act = r["x"].cuda(), r["gm"].cuda(), r["g"].cuda(), r["act"].cuda()
        tag = "layer %d (%s) " % (li + 1, precision)
        _close(capi.conv_forward(x, m, w, b, 9, 1, None, prec), r["pre"], precision, tag + "forward")
        _close(capi.conv_relu_forward(x, m, w, b, 9, 1, None, prec), r["act"], precision, tag + "fused-ReLU forward")
        plan = capi.plan_build(m, None, oh * ow, 9, 1, ih, iw)
        _close(capi.conv_backward_input(gm, plan, w, ih, iw, 9, prec), r["gx"], precision, tag + "dInput")
        gw, gb = capi.conv_backward_weight(gm, x, m, 9, 1, None, prec)
        _close(gw, r["gw"], precision, tag + "dW")
        _close(gb, r["gb"], precision, tag + "dBias")
        _close(capi.conv_relu_backward_input(g, act, plan, w, ih, iw, 9, prec), r["gx"], precision, tag + "fused-ReLU dInput")
        gw, gb = capi.conv_relu_backward_weight(g, act, x, m, 9, 1, None, prec)
        _close(gw, r["gw"], precision, tag + "fused-ReLU dW")
        _close(gb, r["gb"], precision, tag + "fused-ReLU dBias")
        del x, gm, g, act, plan
        torch.cuda.empty_cache()


@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_config4_encoder_stack_small_resolution(precision):
    """The four-layer encoder (config 4) at 32x64 input, batch 2: every operator of every layer against the oracle,
    and the stack driver end to end in the exact precision."""
    from sphmap import capi, workloads as wl
    from sphmap.parallel import EncoderStack
    cfg = wl.config4(B=2, H=32, W=64)
    _check_encoder_per_operator(cfg, precision)
    if precision == "fp32":
        dev = torch.device("cuda:0")
        stack = EncoderStack(cfg, dev, capi.EXACT, 2)
        stack.step(cfg["x"].to(dev), cfg["grad_output"].to(dev))
        L = _encoder_oracle_chain(cfg)
        for li in range(4):
            for name, a, r in (("gw", stack.gw[li], L[li]["gw"]), ("gb", stack.gb[li], L[li]["gb"]), ("gx", stack.gx[li], L[li]["gx"])):
                assert _rel(a.cpu(), r) <= 1e-4, (name, li)
        assert _rel(stack.acts[3].cpu(), L[3]["act"]) <= 1e-5


@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_config4_encoder_stack_full_resolution_per_operator(precision):
    """Config 4 at the resolution the benchmark times (512x1024 input; layers at 256x512 and 128x256 with up to 256
    channels), batch 2.  Layer 4 has 256 pixel tiles per image, so with two images each of the 148 persistent CTAs of
    the tensor-core kernels walks three or four tiles that span both images; the output leaves through the tensor-map
    store at the full strides."""
    from sphmap import workloads as wl
    _check_encoder_per_operator(wl.config4(B=2, H=512, W=1024), precision)


@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_config3_full_resolution_against_oracle(precision):
    """Config 3 at its full resolution (64->128 channels, 256x512, K=9, four weighted nearest points per slot on a
    uniform-random map; transposed conv 128x256 -> 256x512), one image: every operator against the oracle."""
    from sphmap import workloads as wl
    from _gpu_impl import CApi
    o = _oracle()
    c = wl.config3(B=1)
    impl = CApi(precision=1 if precision == "bf16" else 0)
    _close(impl.mapped_conv_forward(c["x"], c["map"], c["weight"], c["bias"], 9, 0, c["iw"]),
           o.mapped_conv_forward(c["x"], c["map"], c["weight"], c["bias"], 9, 0, c["iw"]), precision, "conv forward")
    for name, a, r in zip(("dInput", "dW", "dBias"),
                          impl.mapped_conv_backward(c["grad_output"], c["map"], c["x"], c["weight"], c["bias"], 9, 0, c["iw"]),
                          o.mapped_conv_backward(c["grad_output"], c["map"], c["x"], c["weight"], c["bias"], 9, 0, c["iw"])):
        _close(a, r, precision, "conv " + name)
    t = c["t"]
    _close(impl.mapped_transposed_conv_forward(t["x"], t["map"], t["weight"], t["bias"], t["oh"], t["ow"], 9, 0, t["iw"]),
           o.mapped_transposed_conv_forward(t["x"], t["map"], t["weight"], t["bias"], t["oh"], t["ow"], 9, 0, t["iw"]),
           precision, "tconv forward")
    for name, a, r in zip(("dInput", "dW", "dBias"),
                          impl.mapped_transposed_conv_backward(t["grad_output"], t["map"], t["x"], t["weight"], t["bias"], 9, 0, t["iw"]),
                          o.mapped_transposed_conv_backward(t["grad_output"], t["map"], t["x"], t["weight"], t["bias"], 9, 0, t["iw"])):
        _close(a, r, precision, "tconv " + name)
