"""Fused ReLU (sph_mapped_conv_relu_*): the kernels clamp the forward output and read grad_output * (output > 0) in
backward.  Because masked elements are exactly zero either way, results must be bit-identical to the plain operator
followed by a separate ReLU / masked gradient, on every path (thin kernels, tensor-core kernels, and the fallback
for shapes the library does not fuse)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

CASES = [
    # name, B, Cin, Cout, IH, IW, OH, OW, K, interp, dtype, precision
    ("thin_fp32", 3, 3, 20, 24, 40, 12, 20, 9, 1, torch.float32, "exact"),
    ("thin_fp64", 2, 2, 70, 10, 16, 10, 16, 4, 2, torch.float64, "exact"),
    ("thin_bf16", 2, 3, 64, 32, 64, 16, 32, 9, 1, torch.float32, "bf16"),
    ("tc_bf16", 2, 64, 96, 24, 48, 24, 48, 9, 1, torch.float32, "bf16"),
    ("tc_bf16_down", 2, 64, 128, 32, 64, 8, 16, 9, 1, torch.float32, "bf16"),       # multiply-first adjoint
    ("tc_bf16_odd", 1, 72, 40, 13, 22, 13, 22, 5, 0, torch.float32, "bf16"),         # width not a multiple of 4
    ("fallback_exact", 2, 8, 12, 12, 20, 12, 20, 9, 1, torch.float32, "exact"),       # SIMT GEMM: not fused
]


def _inputs(c):
    name, B, Cin, Cout, IH, IW, OH, OW, K, interp, dtype, prec = c
    g = torch.Generator().manual_seed(hash(name) % 1000)
    x = torch.randn(B, Cin, IH, IW, generator=g, dtype=dtype).cuda()
    w = (torch.randn(Cout, Cin, K, generator=g, dtype=dtype) / (Cin * K) ** 0.5).cuda()
    b = (torch.randn(Cout, generator=g, dtype=dtype) * 0.1).cuda()
    m = (torch.rand(OH, OW, K, 2, generator=g, dtype=dtype) * torch.tensor([IW + 1.0, IH + 1.0], dtype=dtype) - 1).cuda()
    go = torch.randn(B, Cout, OH, OW, generator=g, dtype=dtype).cuda()
    return x, w, b, m, go


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_c_abi_fused_equals_unfused(case):
    from sphmap import capi
    name, B, Cin, Cout, IH, IW, OH, OW, K, interp, dtype, prec = case
    p = capi.BF16 if prec == "bf16" else capi.EXACT
    x, w, b, m, go = _inputs(case)
    y_ref = capi.conv_forward(x, m, w, b, K, interp, precision=p).clamp_(min=0)
    y = capi.conv_relu_forward(x, m, w, b, K, interp, precision=p)
    assert torch.equal(y, y_ref)
    assert (y == 0).any() and (y > 0).any()
    plan = capi.plan_build(m, None, OH * OW, K, interp, IH, IW)
    gm = go * (y > 0)
    gx_ref = capi.conv_backward_input(gm, plan, w, IH, IW, K, precision=p)
    gw_ref, gb_ref = capi.conv_backward_weight(gm, x, m, K, interp, precision=p)
    gx = capi.conv_relu_backward_input(go, y, plan, w, IH, IW, K, precision=p)
    gw, gb = capi.conv_relu_backward_weight(go, y, x, m, K, interp, precision=p)
    assert torch.equal(gx, gx_ref)
    assert torch.equal(gw, gw_ref)
    assert torch.equal(gb, gb_ref)


def test_fused_entry_points_refuse_what_they_do_not_fuse():
    from sphmap import capi
    case = CASES[-1]
    name, B, Cin, Cout, IH, IW, OH, OW, K, interp, dtype, prec = case
    x, w, b, m, go = _inputs(case)
    out = torch.empty(B, Cout, OH, OW, dtype=dtype, device="cuda")
    ws = capi.conv_workspace(capi.CONV_FORWARD, B, Cin, Cout, IH, IW, OH, OW, K, 0, capi.F32, interp, capi.EXACT, x)
    rc = capi.lib.sph_mapped_conv_relu_forward(capi._ptr(x), capi._ptr(m), capi._ptr(None), capi._ptr(w), capi._ptr(b),
                                               capi._ptr(out), *capi._ints(B, Cin, Cout, IH, IW, OH, OW, K, 0),
                                               capi._int(capi.F32), capi._int(interp), capi._int(capi.EXACT),
                                               capi._ptr(ws[0]), capi._sz(ws[1]), capi._stream())
    assert rc == capi.ERR_UNSUPPORTED


@pytest.mark.parametrize("precision", ["fp32", "bf16"])
def test_layer_with_fused_activation_matches_layer_plus_relu(precision):
    import _spherical_distortion_ext._C as C
    from spherical_distortion.nn import InterpolationType, MappedConvolution
    old = C.get_precision()
    C.set_precision(precision)
    try:
        g = torch.Generator().manual_seed(3)
        for cin, cout in ((3, 32), (64, 64)):
            x = torch.randn(2, cin, 16, 32, generator=g).cuda().requires_grad_(True)
            m = (torch.rand(16, 32, 9, 2, generator=g) * torch.tensor([32.0, 16.0]) - 0.5).cuda()
            plain = MappedConvolution(cin, cout, 9, InterpolationType.BILINEAR).cuda()
            fused = MappedConvolution(cin, cout, 9, InterpolationType.BILINEAR, activation="relu").cuda()
            fused.load_state_dict(plain.state_dict())
            go = torch.randn(2, cout, 16, 32, generator=g).cuda()
            y0 = torch.relu(plain(x, m))
            y0.backward(go)
            gx0, gw0, gb0 = x.grad.clone(), plain.weight.grad.clone(), plain.bias.grad.clone()
            x.grad = None
            y1 = fused(x, m)
            y1.backward(go)
            assert torch.equal(y1, y0)
            assert torch.equal(x.grad, gx0)
            assert torch.equal(fused.weight.grad, gw0)
            assert torch.equal(fused.bias.grad, gb0)
    finally:
        C.set_precision(old)


@pytest.mark.parametrize("level", ["c_abi", "layer"])
def test_weighted_bilinear_three_points_bf16(level):
    """Weighted bilinear map with three points per slot (12 taps), 64 channels, bf16: the gather-GEMM fuses the mask,
    the weight-gradient kernel declines (its tap table is the smaller one), and each side must fall back on its own
    with results identical to the unfused composition."""
    import _spherical_distortion_ext._C as C
    from sphmap import capi
    from spherical_distortion.nn import InterpolationType, MappedConvolution
    g = torch.Generator().manual_seed(17)
    B, Cin, Cout, H, W, K, P = 2, 64, 48, 12, 24, 9, 3
    x = torch.randn(B, Cin, H, W, generator=g).cuda()
    m = (torch.rand(H, W, K, P, 2, generator=g) * torch.tensor([W + 1.0, H + 1.0]) - 1).cuda()
    iw = torch.rand(H, W, K, P, generator=g).cuda()
    go = torch.randn(B, Cout, H, W, generator=g).cuda()
    if level == "c_abi":
        w = (torch.randn(Cout, Cin, K, generator=g) / (Cin * K) ** 0.5).cuda()
        b = (torch.randn(Cout, generator=g) * 0.1).cuda()
        y = capi.conv_relu_forward(x, m, w, b, K, 1, iw, capi.BF16)
        assert torch.equal(y, capi.conv_forward(x, m, w, b, K, 1, iw, capi.BF16).clamp_(min=0))
        plan = capi.plan_build(m, iw, H * W, K, 1, H, W)
        gm = go * (y > 0)
        assert torch.equal(capi.conv_relu_backward_input(go, y, plan, w, H, W, K, capi.BF16),
                           capi.conv_backward_input(gm, plan, w, H, W, K, capi.BF16))
        got, want = capi.conv_relu_backward_weight(go, y, x, m, K, 1, iw, capi.BF16), capi.conv_backward_weight(gm, x, m, K, 1, iw, capi.BF16)
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
        return
    old = C.get_precision()
    C.set_precision("bf16")
    try:
        x.requires_grad_(True)
        plain = MappedConvolution(Cin, Cout, K, InterpolationType.BILINEAR).cuda()
        fused = MappedConvolution(Cin, Cout, K, InterpolationType.BILINEAR, activation="relu").cuda()
        fused.load_state_dict(plain.state_dict())
        y0 = torch.relu(plain(x, m, iw))
        y0.backward(go)
        gx0 = x.grad.clone()
        x.grad = None
        y1 = fused(x, m, iw)
        y1.backward(go)
        assert torch.equal(y1, y0) and torch.equal(x.grad, gx0)
        assert torch.equal(fused.weight.grad, plain.weight.grad) and torch.equal(fused.bias.grad, plain.bias.grad)
    finally:
        C.set_precision(old)


def test_encoder_stack_fused_equals_unfused():
    from sphmap import capi, workloads as wl
    from sphmap.parallel import EncoderStack
    cfg = wl.config4(B=2, H=64, W=128)
    dev = torch.device("cuda")
    x, go = cfg["x"].to(dev), cfg["grad_output"].to(dev)
    res = []
    for fuse in (False, True):
        st = EncoderStack(cfg, dev, capi.BF16, 2, fuse_relu=fuse)
        loss = st.step(x, go)
        res.append((loss.clone(), [t.clone() for t in st.gw], [t.clone() for t in st.gb], st.gx[0].clone()))
    assert torch.equal(res[0][0], res[1][0])
    for a, b in zip(res[0][1] + res[0][2] + [res[0][3]], res[1][1] + res[1][2] + [res[1][3]]):
        assert torch.equal(a, b)


def test_companions_and_combined_backward_are_bit_identical_to_the_separate_calls():
    """Channels-last companions (written by a layer's epilogue, gathered from by the next layer) and the combined
    backward call (grad_output converted once for dInput and dW) change where the bf16 copies come from, not their
    contents: every result equals the plain entry points' bit for bit."""
    from sphmap import capi, workloads as wl
    g = torch.Generator().manual_seed(91)
    B, C0, C1, C2, H, W, K = 2, 3, 64, 128, 32, 64, 9
    x = torch.rand(B, C0, H, W, generator=g).cuda()
    m1, m2 = wl.gnomonic_map(H, W, 2).cuda(), wl.gnomonic_map(H // 2, W // 2, 1).cuda()
    w1, b1 = (torch.randn(C1, C0, K, generator=g) / 5).cuda(), (torch.randn(C1, generator=g) * 0.1).cuda()
    w2, b2 = (torch.randn(C2, C1, K, generator=g) / 24).cuda(), (torch.randn(C2, generator=g) * 0.1).cuda()
    go = torch.randn(B, C2, H // 2, W // 2, generator=g).cuda()
    # plain path
    a1 = capi.conv_relu_forward(x, m1, w1, b1, K, 1, None, capi.BF16)
    a2 = capi.conv_relu_forward(a1, m2, w2, b2, K, 1, None, capi.BF16)
    plan2 = capi.plan_build(m2, None, (H // 2) * (W // 2), K, 1, H // 2, W // 2)
    gx_ref = capi.conv_relu_backward_input(go, a2, plan2, w2, H // 2, W // 2, K, capi.BF16)
    gw_ref, gb_ref = capi.conv_relu_backward_weight(go, a2, a1, m2, K, 1, None, capi.BF16)
    # companions: layer 1 (thin kernels) writes the companion of its output, layer 2 (tensor cores) gathers from it
    cl1 = capi.companion(B, C1, H // 2, W // 2, "cuda")
    cl2 = capi.companion(B, C2, H // 2, W // 2, "cuda")
    c1 = capi.conv_forward_cl(x, None, m1, w1, b1, K, 1, None, capi.BF16, True, out_cl=cl1)
    c2 = capi.conv_forward_cl(c1, cl1, m2, w2, b2, K, 1, None, capi.BF16, True, out_cl=cl2)
    assert torch.equal(c1, a1) and torch.equal(c2, a2)
    # the companion holds bf16(activation), channels last, with a zero pixel behind every image
    n1 = (H // 2) * (W // 2)
    v = cl1[:B * (n1 + 1) * C1 * 2].view(torch.bfloat16).view(B, n1 + 1, C1)
    assert torch.equal(v[:, :n1].float(), a1.to(torch.bfloat16).float().flatten(2).transpose(1, 2)) and (v[:, n1] == 0).all()
    gx, gw, gb = capi.conv_backward_cl(go, c2, c1, cl1, plan2, m2, w2, K, 1, None, capi.BF16)
    assert torch.equal(gx, gx_ref) and torch.equal(gw, gw_ref) and torch.equal(gb, gb_ref)
    gx, gw, gb = capi.conv_backward_cl(go, c2, c1, None, plan2, m2, w2, K, 1, None, capi.BF16)      # without the companion of x
    assert torch.equal(gx, gx_ref) and torch.equal(gw, gw_ref) and torch.equal(gb, gb_ref)
    gx, gw, gb = capi.conv_backward_cl(go * (c2 > 0), None, c1, cl1, plan2, m2, w2, K, 1, None, capi.BF16)   # unfused mask
    assert torch.equal(gx, gx_ref) and torch.equal(gw, gw_ref) and torch.equal(gb, gb_ref)
    # a thin layer (3 input channels) has its own combined kernel in bf16 precision: same results as its separate
    # entry points; the exact precision declines the combined call before launching anything
    plan1 = capi.plan_build(m1, None, n1, K, 1, H, W)
    tx, tw, tb = capi.conv_backward_cl(gx_ref, a1, x, None, plan1, m1, w1, K, 1, None, capi.BF16)
    assert torch.equal(tx, capi.conv_relu_backward_input(gx_ref, a1, plan1, w1, H, W, K, capi.BF16))
    sw, sb = capi.conv_relu_backward_weight(gx_ref, a1, x, m1, K, 1, None, capi.BF16)
    assert torch.equal(tw, sw) and torch.equal(tb, sb)
    with pytest.raises(capi.Unsupported):
        capi.conv_backward_cl(gx_ref, a1, x, None, plan1, m1, w1, K, 1, None, capi.EXACT)
    # ragged sizes (tiles with tail pixels, width not a multiple of 4 -> plain-store epilogue) and a down-sampling map
    xr = torch.randn(1, 72, 13, 22, generator=g).cuda()
    mr = (torch.rand(13, 22, 5, 2, generator=g) * torch.tensor([23.0, 14.0]) - 0.5).cuda()
    wr, br = (torch.randn(40, 72, 5, generator=g) / 19).cuda(), torch.zeros(40).cuda()
    clr = capi.companion(1, 40, 13, 22, "cuda")
    yr = capi.conv_forward_cl(xr, None, mr, wr, br, 5, 1, None, capi.BF16, True, out_cl=clr)
    assert torch.equal(yr, capi.conv_relu_forward(xr, mr, wr, br, 5, 1, None, capi.BF16))
    cp = 64   # 40 channels pad to 64
    vr = clr[:(13 * 22 + 1) * cp * 2].view(torch.bfloat16).view(13 * 22 + 1, cp)
    assert torch.equal(vr[:13 * 22, :40].float(), yr.to(torch.bfloat16).float().flatten(2)[0].t()) and (vr[:, 40:] == 0).all()


def test_encoder_stack_with_companions_equals_without():
    from sphmap import capi, workloads as wl
    from sphmap.parallel import EncoderStack
    cfg = wl.config4(B=2, H=64, W=128)
    dev = torch.device("cuda")
    x, go = cfg["x"].to(dev), cfg["grad_output"].to(dev)
    res = []
    for comp in (False, True):
        st = EncoderStack(cfg, dev, capi.BF16, 2, companions=comp)
        for _ in range(2):      # twice: the companions are reused across steps
            loss = st.step(x, go)
        res.append((loss.clone(), [t.clone() for t in st.gw], [t.clone() for t in st.gb], st.gx[0].clone()))
        assert any(st.combined) == comp
    assert torch.equal(res[0][0], res[1][0])
    for a, b in zip(res[0][1] + res[0][2] + [res[0][3]], res[1][1] + res[1][2] + [res[1][3]]):
        assert torch.equal(a, b)


def test_encoder_stack_writes_gradients_into_the_reducer_buffers():
    """With a gradient reducer the stack's dW and dBias of a layer are adjacent views of one flat buffer that the
    kernels write directly (the allreduce then runs on it in place): same values as with separately allocated
    gradients, in both precisions."""
    from sphmap import capi, workloads as wl
    from sphmap.parallel import EncoderStack, GradReducer
    cfg = wl.config4(B=2, H=64, W=128)
    dev = torch.device("cuda")
    x, go = cfg["x"].to(dev), cfg["grad_output"].to(dev)
    for prec in (capi.BF16, capi.EXACT):
        res = []
        for red in (None, GradReducer()):
            st = EncoderStack(cfg, dev, prec, 2, reducer=red)
            ptrs = [t.data_ptr() for t in st.gw]
            for _ in range(2):
                st.step(x, go)
            assert [t.data_ptr() for t in st.gw] == ptrs       # fixed buffers, step after step
            if red is not None:
                assert all(b.data_ptr() == w.data_ptr() + 4 * w.numel() for w, b in zip(st.gw, st.gb))
            res.append([t.clone() for t in st.gw + st.gb])
        for a, b in zip(*res):
            assert torch.equal(a, b)


def test_layer_stack_with_and_without_companion_cache():
    """Two stacked layers with the fused activation through the module API in bf16: with the companion cache on, the
    second layer gathers from the channels-last copy the first one left; results and gradients equal the run with the
    cache off bit for bit, also when the intermediate tensor was modified in place (the stale copy must not be used)."""
    import _spherical_distortion_ext as ext
    from spherical_distortion.nn import InterpolationType, MappedConvolution
    from sphmap import workloads as wl
    old = ext.get_precision()
    ext.set_precision("bf16")
    try:
        g = torch.Generator().manual_seed(77)
        x = torch.rand(2, 3, 32, 64, generator=g).cuda().requires_grad_(True)
        m1, m2 = wl.gnomonic_map(32, 64, 2).cuda(), wl.gnomonic_map(16, 32, 1).cuda()
        l1 = MappedConvolution(3, 64, 9, InterpolationType.BILINEAR, activation="relu").cuda()
        l2 = MappedConvolution(64, 96, 9, InterpolationType.BILINEAR, activation="relu").cuda()
        go = torch.randn(2, 96, 16, 32, generator=g).cuda()
        runs = []
        for on in (False, True):
            ext.set_companions(on)
            for p in list(l1.parameters()) + list(l2.parameters()) + [x]:
                p.grad = None
            y = l2(l1(x, m1), m2)
            y.backward(go)
            runs.append([y.detach().clone(), x.grad.clone()] + [p.grad.clone() for p in list(l1.parameters()) + list(l2.parameters())])
        for a, b in zip(runs[0], runs[1]):
            assert torch.equal(a, b)
        # a tensor modified in place after the layer produced it no longer matches its cached copy (version counter):
        # the next layer converts the tensor itself instead of gathering from the stale copy
        ext.set_companions(True)
        with torch.no_grad():
            h = l1(x, m1)
            h.add_(0.25)
            y_inplace = l2(h, m2)
            y_fresh = l2(h.clone(), m2)
        assert torch.equal(y_inplace, y_fresh)
    finally:
        ext.set_companions(True)
        ext.set_precision(old)


def test_unfused_composition_converts_an_input_once():
    """The reference's own composition (convolution, then a separate torch.relu) in bf16 precision: no layer leaves a
    channels-last copy for the next one, so the host extension converts a layer's input once in forward and keeps the
    copy for the weight gradient in backward.  Results and gradients equal the run with the cache off bit for bit, and
    sph_conv_companion_fill writes what a fused forward would have written."""
    import _spherical_distortion_ext as ext
    from spherical_distortion.nn import InterpolationType, MappedConvolution
    from sphmap import capi, workloads as wl
    old = ext.get_precision()
    ext.set_precision("bf16")
    try:
        g = torch.Generator().manual_seed(78)
        x = torch.rand(2, 3, 32, 64, generator=g).cuda().requires_grad_(True)
        m1, m2 = wl.gnomonic_map(32, 64, 2).cuda(), wl.gnomonic_map(16, 32, 1).cuda()
        l1 = MappedConvolution(3, 64, 9, InterpolationType.BILINEAR).cuda()
        l2 = MappedConvolution(64, 96, 9, InterpolationType.BILINEAR).cuda()
        go = torch.randn(2, 96, 16, 32, generator=g).cuda()
        runs = []
        for on in (False, True):
            ext.set_companions(on)
            for p in list(l1.parameters()) + list(l2.parameters()) + [x]:
                p.grad = None
            y = l2(torch.relu(l1(x, m1)), m2)
            y.backward(go)
            runs.append([y.detach().clone(), x.grad.clone()] + [p.grad.clone() for p in list(l1.parameters()) + list(l2.parameters())])
        for a, b in zip(runs[0], runs[1]):
            assert torch.equal(a, b)
    finally:
        ext.set_companions(True)
        ext.set_precision(old)
    # the entry point itself: the same bytes as the copy a fused forward writes beside its output
    xa = torch.rand(2, 16, 8, 16, generator=torch.Generator().manual_seed(5)).cuda()
    ma = wl.gnomonic_map(8, 16, 1).cuda()
    wa, ba = (torch.randn(64, 16, 9) / 12).cuda(), torch.zeros(64).cuda()
    cl = capi.companion(2, 64, 8, 16, "cuda")
    out = capi.conv_forward_cl(xa, None, ma, wa, ba, 9, 1, None, capi.BF16, True, out_cl=cl)
    assert torch.equal(capi.companion_of(out), cl)
