"""Operators beside the convolution path that share its kernels, on the GPU: mapped average pooling and its backward,
UV-map gather / scatter, voting resampling, the normalised scatter, the deterministic argmax backward, the device
map builders and the standard-convolution wrappers.  Checked against the golden vectors produced by the reference's
compiled CPU modules (tests/golden/reference_siblings.pt) and against the CPU oracle on larger seeded cases.
Gathers are bit exact; scatters (the reference adds with atomics, this library in map order) within
1e-5 * max|ref| in float32 and 1e-12 in float64."""
import os

import pytest
import torch

from oracle import port

pytestmark = pytest.mark.gpu


def _golden(golden_dir):
    return torch.load(os.path.join(golden_dir, "reference_siblings.pt"), weights_only=False)


def _close(a, b):
    a, b = a.cpu(), b.cpu()
    tol = 1e-5 if b.dtype == torch.float32 else 1e-12
    torch.testing.assert_close(a, b, rtol=tol, atol=tol * max(1.0, b.abs().max().item()))


def _cuda(*ts):
    return [None if t is None else t.cuda() for t in ts]


@pytest.mark.parametrize("level", ["c_abi", "plugin"])
def test_siblings_match_reference_golden_vectors(golden_dir, level):
    from sphmap import capi
    import _spherical_distortion_ext._C as C
    n = 0
    for c in _golden(golden_dir):
        if c["op"] == "avgpool":
            x, m, iw, g = _cuda(c["input"], c["sample_map"], c["interp_weights"], c["grad_output"])
            K, it = c["kernel_size"], c["interp"]
            IH, IW = x.shape[2:]
            if level == "c_abi":
                out = capi.mapped_avg_pool(x, m, K, it, iw)
                gin = capi.mapped_avg_unpool(g, capi.slot_plan_build(m, iw, K, it, IH, IW), IH, IW, K)
            elif iw is None:
                out = C.mapped_avg_pool(x, m, K, C.InterpolationType(it))
                gin = C.mapped_avg_unpool(g, m, torch.tensor(IH), torch.tensor(IW), torch.tensor(K), C.InterpolationType(it))
            else:
                out = C.weighted_mapped_avg_pool(x, m, iw, K, C.InterpolationType(it))
                gin = C.weighted_mapped_avg_unpool(g, m, iw, IH, IW, K, C.InterpolationType(it))
            assert torch.equal(out.cpu(), c["ref_output"]), ("avgpool", c["seed"], it)
            _close(gin, c["ref_grads"][0])
        elif c["op"] == "uv":
            tex, quad, uv, img = _cuda(c["input"], c["quad_idx"], c["tex_uv"], c["grad_output"])
            it = c["interp"]
            NT, TH, TW = tex.shape[2:]
            if level == "c_abi":
                out = capi.resample_from_uv_maps(tex, quad, uv, it)
                back = capi.resample_to_uv_maps(img, quad, uv, NT, TH, TW, it)
            else:
                out = C.resample_from_uv_maps(tex, quad, uv, C.InterpolationType(it))
                back = C.resample_to_uv_maps(img, quad, uv, NT, TH, TW, C.InterpolationType(it))
            assert torch.equal(out.cpu(), c["ref_output"]), ("uv", c["seed"], it)
            _close(back, c["ref_grads"][0])
        elif c["op"] == "voting":
            lab, m = _cuda(c["input"], c["sample_map"])
            fn = capi.voting_resample_to_map if level == "c_abi" else C.voting_resample_to_map
            assert torch.equal(fn(lab, m, c["oh"], c["ow"], c["num_candidates"]).cpu(), c["ref_output"]), c["seed"]
        else:
            continue
        n += 1
    assert n == 21


def test_device_map_builders_match_the_reference_python_builders(golden_dir):
    """Against the reference's own builders: to float64 round-off in float64; the float32 maps of the reference are
    evaluated in float32 throughout and differ from a float64 evaluation by up to ~1e-3 px."""
    import spherical_distortion.util as u
    fns = {"grid": u.grid_projection_map, "inverse_gnomonic": u.inverse_gnomonic_projection_map,
           "inverse_equirectangular": u.inverse_equirectangular_projection_map}
    n = 0
    for c in _golden(golden_dir):
        if c["op"] != "map":
            continue
        args = ((c["H"], c["W"]), (c["kh"], c["kw"]), c["stride"], c["dilation"])
        m64 = fns[c["kind"]](*args, dtype=torch.float64).cpu()
        m32 = fns[c["kind"]](*args).cpu()
        assert m64.shape == c["f64"].shape and m32.dtype == torch.float32
        ok = ~torch.isnan(c["f64"])   # even kernels: the reference's zero differential is 0/0; here it is the pixel itself
        assert torch.isfinite(m64).all()
        # A sample whose own latitude is a pole has no defined longitude: its x comes out of a division by, or the sign
        # of, cos(+-pi/2) (+6e-17 in float64, -4e-8 in float32), i.e. of round-off.  Those samples are compared in y
        # only; on the two pole rows the same holds for every tangent-plane sample of the float32 maps.
        y = c["f64"][..., 1:2]
        defined = ok & (y > 1e-6) & (y < c["H"] - 1 - 1e-6)
        # longitudes within round-off of the +-pi seam may wrap to either end of the row: compare x modulo W
        d = (m64 - c["f64"]).abs()
        d[..., 0] = torch.minimum(d[..., 0], (d[..., 0] - c["W"]).abs())
        assert d[defined].max() <= 1e-9 and d[..., 1][ok[..., 1]].max() <= 1e-9, (c["kind"], d[defined].max())
        d32 = (m32.double() - c["f32"].double()).abs()
        d32[..., 0] = torch.minimum(d32[..., 0], (d32[..., 0] - c["W"]).abs())
        rows = torch.arange(0, c["H"], c["stride"])
        defined32 = defined & ((rows != 0) & (rows != c["H"] - 1)).view(-1, 1, 1, 1)
        assert d32[defined32].max() <= 2e-3 and d32[..., 1][ok[..., 1]].max() <= 2e-3, (c["kind"], d32[defined32].max())
        n += 1
    assert n == 12
    # a map built on the device drives a layer exactly like the same map built on the host
    from sphmap import workloads as wl
    dev_map = u.inverse_gnomonic_projection_map((64, 128), (3, 3), 2)
    host_map = wl.gnomonic_map(64, 128, 2).cuda()
    assert (dev_map - host_map).abs().max() <= 1e-3


@pytest.mark.parametrize("interp,P,dtype", [(0, 0, torch.float32), (1, 0, torch.float32), (2, 3, torch.float64), (1, 2, torch.float32)])
def test_deterministic_argmax_backward(interp, P, dtype):
    """sph_mapped_max_unpool_planned against the oracle and the atomic kernel, and run twice for bit identity; many
    outputs collide on each input pixel (down-sampling map) so the summation order matters."""
    from sphmap import capi
    g = torch.Generator().manual_seed(10 + interp + P)
    B, C, IH, IW, OH, OW, K = 3, 5, 12, 20, 24, 40, 9
    x = torch.randn(B, C, IH, IW, generator=g, dtype=dtype)
    shape = (OH, OW, K, P, 2) if P else (OH, OW, K, 2)
    m = (torch.rand(*shape, generator=g, dtype=torch.float64) * torch.tensor([IW + 1.0, IH + 1.0]) - 1.0).to(dtype)
    iw = torch.rand(OH, OW, K, P, generator=g, dtype=dtype) if P else None
    go = torch.randn(B, C, OH, OW, generator=g, dtype=dtype)
    xd, md, iwd, god = _cuda(x, m, iw, go)
    out, idx = capi.mapped_max_pool(xd, md, K, interp, iwd)
    plan = capi.slot_plan_build(md, iwd, K, interp, IH, IW)
    a = capi.mapped_max_unpool_planned(god, idx, plan, IH, IW, K, P)
    b = capi.mapped_max_unpool_planned(god, idx, plan, IH, IW, K, P)
    assert torch.equal(a, b)
    _close(a, capi.mapped_max_unpool(god, idx, md, IH, IW, K, interp, iwd))
    _close(a, port.mapped_max_unpool(go, idx.cpu(), m, IH, IW, K, interp, iw))
    # outputs without a winner (index -1) contribute nothing
    idx2 = idx.clone()
    idx2[:, :, ::2] = -1
    god2 = god.clone()
    god2[:, :, ::2] = 0
    assert torch.equal(capi.mapped_max_unpool_planned(god, idx2, plan, IH, IW, K, P),
                       capi.mapped_max_unpool_planned(god2, idx, plan, IH, IW, K, P))


def test_deterministic_argmax_backward_without_staging():
    """More outputs per plane than the shared-memory staging holds: the kernel reads idx from global memory."""
    from sphmap import capi
    g = torch.Generator().manual_seed(3)
    B, C, IH, IW, OH, OW, K = 1, 2, 64, 128, 256, 256, 4
    x = torch.randn(B, C, IH, IW, generator=g)
    m = torch.rand(OH, OW, K, 2, generator=g) * torch.tensor([float(IW), float(IH)])
    go = torch.randn(B, C, OH, OW, generator=g)
    xd, md, god = _cuda(x, m, go)
    out, idx = capi.mapped_max_pool(xd, md, K, 1)
    plan = capi.slot_plan_build(md, None, K, 1, IH, IW)
    a = capi.mapped_max_unpool_planned(god, idx, plan, IH, IW, K)
    assert torch.equal(a, capi.mapped_max_unpool_planned(god, idx, plan, IH, IW, K))
    _close(a, port.mapped_max_unpool(go, idx.cpu(), m, IH, IW, K, 1))


def test_layer_argmax_backward_is_deterministic_by_default():
    from spherical_distortion.nn import InterpolationType, MappedMaxPool
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 4, 16, 32, generator=g).cuda().requires_grad_(True)
    m = (torch.rand(32, 64, 9, 2, generator=g) * torch.tensor([32.0, 16.0])).cuda()
    go = torch.randn(2, 4, 32, 64, generator=g).cuda()
    grads = []
    for _ in range(2):
        x.grad = None
        MappedMaxPool(9, InterpolationType.BILINEAR)(x, m).backward(go)
        grads.append(x.grad.clone())
    assert torch.equal(grads[0], grads[1])


@pytest.mark.parametrize("interp,P", [(1, 0), (0, 0), (2, 2)])
def test_normalised_scatter_equals_scatter_over_scattered_ones(interp, P):
    from sphmap import capi
    from spherical_distortion import functional as F
    from spherical_distortion.nn import InterpolationType
    g = torch.Generator().manual_seed(21 + interp)
    B, C, MH, MW, OH, OW = 2, 3, 40, 24, 32, 64
    x = torch.randn(B, C, MH, MW, generator=g)
    shape = (MH, MW, P, 2) if P else (MH, MW, 2)
    m = torch.rand(*shape, generator=g) * torch.tensor([OW + 1.0, OH + 1.0]) - 1.0
    iw = torch.rand(MH, MW, P, generator=g) if P else None
    xd, md, iwd = _cuda(x, m, iw)
    plan = capi.plan_build(md, iwd, MH * MW, 1, interp, OH, OW)
    fused = capi.resample_to_map_normalized(xd, plan, OH, OW)
    ones = torch.ones(1, 1, MH, MW, device="cuda")
    composed = capi.resample_to_map(xd, plan, OH, OW) / (capi.resample_to_map(ones, plan, OH, OW) + 1e-12)
    assert torch.equal(fused, composed)
    want = port.resample_to_map(x, m, OH, OW, interp, iw) / (port.resample_to_map(ones.cpu(), m, OH, OW, interp, iw) + 1e-12)
    torch.testing.assert_close(fused.cpu(), want, rtol=1e-4, atol=1e-5 * want.abs().max().item())
    assert torch.equal(F.resample_normalized(xd, md, (OH, OW), InterpolationType(interp), iwd), fused)


def test_average_pool_layer_gradcheck_and_larger_case():
    from sphmap import capi
    from spherical_distortion.nn import InterpolationType, MappedAvgPool, MappedAvgUnpool
    g = torch.Generator().manual_seed(31)
    x = torch.randn(1, 2, 5, 6, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    m = (torch.rand(3, 4, 4, 2, generator=g, dtype=torch.float64) * torch.tensor([6.0, 5.0]) - 0.5).cuda()
    assert torch.autograd.gradcheck(lambda t: MappedAvgPool(4, InterpolationType.BILINEAR)(t, m), (x,))
    y = torch.randn(1, 2, 3, 4, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    assert torch.autograd.gradcheck(lambda t: MappedAvgUnpool(4, InterpolationType.BILINEAR)(t, 5, 6, m), (y,))
    # a pooling layer of a spherical network: 64 planes, 3x3 gnomonic map with stride 2
    from sphmap import workloads as wl
    xb = torch.randn(2, 32, 64, 128, generator=g)
    mb = wl.gnomonic_map(64, 128, 2)
    got = capi.mapped_avg_pool(xb.cuda(), mb.cuda(), 9, 1)
    assert torch.equal(got.cpu(), port.mapped_avg_pool(xb, mb, 9, 1))
    gb = torch.randn(2, 32, 32, 64, generator=g)
    gin = capi.mapped_avg_unpool(gb.cuda(), capi.slot_plan_build(mb.cuda(), None, 9, 1, 64, 128), 64, 128, 9)
    _close(gin, port.mapped_avg_unpool(gb, mb, 64, 128, 9, 1))


def test_uv_resample_layer_gradcheck_and_tangent_round_trip():
    from spherical_distortion import functional as F
    from spherical_distortion.nn import InterpolationType, ResampleFromUV
    g = torch.Generator().manual_seed(41)
    tex = torch.randn(1, 2, 3, 4, 5, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    quad = torch.randint(0, 3, (6, 7), generator=g).cuda()
    uv = (torch.rand(6, 7, 2, generator=g, dtype=torch.float64) * torch.tensor([5.0, 4.0]) - 0.5).cuda()
    assert torch.autograd.gradcheck(lambda t: ResampleFromUV(InterpolationType.BILINEAR)(t, quad, uv), (tex,))
    # tangent images and back: faces addressed through the UV maps reproduce what the sample map gathered
    x = torch.randn(2, 3, 16, 32, generator=g).cuda()
    smap = (torch.rand(4, 9, 2, generator=g) * torch.tensor([31.0, 15.0])).cuda()       # 4 faces of 3 x 3 samples
    t = F.create_tangent_images(x, smap, 3, InterpolationType.BILINEAR)
    assert tuple(t.shape) == (2, 3, 4, 3, 3)
    q = torch.randint(0, 4, (16, 32), generator=g).cuda()
    uv2 = (torch.rand(16, 32, 2, generator=g) * 2.0).cuda()
    back = F.tangent_images_to_equirectangular(t, q, uv2, InterpolationType.BILINEAR)
    assert torch.equal(back.cpu(), port.resample_from_uv_maps(t.cpu(), q.cpu(), uv2.cpu(), 1))


def test_voting_resample_many_to_one_and_multi_channel():
    from spherical_distortion import functional as F
    g = torch.Generator().manual_seed(51)
    lab = torch.randint(0, 7, (2, 3, 32, 48), generator=g)
    m = torch.stack((torch.randint(-2, 10, (32, 48), generator=g), torch.randint(-2, 8, (32, 48), generator=g)), -1)
    want = port.voting_resample_to_map(lab, m, 6, 8, 7)
    got = F.voting_resample(lab.cuda(), m.cuda(), None, (6, 8), 7)
    assert torch.equal(got.cpu(), want)


def test_standard_convolution_wrappers_match_torch():
    """The plain convolution layers of the reference package (not mapped operators) delegate to ATen; same results
    and gradients as torch.nn.functional with the reference layers' parameter shapes."""
    import torch.nn.functional as TF
    from spherical_distortion.nn import Convolution, TransposedConvolution
    g = torch.Generator().manual_seed(61)
    x = torch.randn(2, 3, 9, 11, generator=g, dtype=torch.float64).cuda().requires_grad_(True)
    conv = Convolution(3, 5, (3, 2), stride=(2, 1), padding=(1, 0), dilation=(1, 2)).double().cuda()
    y = conv(x)
    ref = TF.conv2d(x, conv.weight, conv.bias, (2, 1), (1, 0), (1, 2))
    torch.testing.assert_close(y, ref)
    go = torch.randn_like(y)
    gx, gw, gb = torch.autograd.grad(y, (x, conv.weight, conv.bias), go)
    rx, rw, rb = torch.autograd.grad(ref, (x, conv.weight, conv.bias), go)
    for a, b in ((gx, rx), (gw, rw), (gb, rb)):
        torch.testing.assert_close(a, b)
    tconv = TransposedConvolution(3, 4, 3, stride=2, padding=1).double().cuda()
    assert tuple(tconv.weight.shape) == (3, 4, 3, 3)
    yt = tconv(x)
    reft = TF.conv_transpose2d(x, tconv.weight, tconv.bias, 2, 1)
    torch.testing.assert_close(yt, reft)
    got = torch.randn_like(yt)
    for a, b in zip(torch.autograd.grad(yt, (x, tconv.weight, tconv.bias), got), torch.autograd.grad(reft, (x, tconv.weight, tconv.bias), got)):
        torch.testing.assert_close(a, b)


def test_plan_with_very_long_segments():
    """A map that sends thousands of samples to a handful of pixels: the plan's per-pixel ordering takes the heap-sort
    path; the scatter still sums every pixel in map order (compared with a float64 sum taken in that order)."""
    from sphmap import capi
    g = torch.Generator().manual_seed(71)
    MH, MW, OH, OW = 64, 96, 8, 8
    m = torch.zeros(MH, MW, 2)
    m[..., 0] = torch.randint(2, 5, (MH, MW), generator=g).float()      # x in {2, 3, 4}
    m[..., 1] = 3.0
    x = torch.randn(2, 2, MH, MW, generator=g)
    plan = capi.plan_build(m.cuda(), None, MH * MW, 1, 0, OH, OW)
    out = capi.resample_to_map(x.cuda(), plan, OH, OW)
    assert torch.equal(out, capi.resample_to_map(x.cuda(), plan, OH, OW))
    want = port.resample_to_map(x, m, OH, OW, 0)
    torch.testing.assert_close(out.cpu(), want, rtol=1e-4, atol=1e-4 * want.abs().max().item())
    # in-order float32 sum of one pixel, reproduced on the host
    sel = (m[..., 0] == 3.0).flatten()
    acc = torch.zeros((), dtype=torch.float32)
    for v in x[0, 0].flatten()[sel]:
        acc = acc + v
    assert out[0, 0, 3, 3].item() == acc.item()


def test_plan_cache_under_inference_mode_and_across_streams():
    import _spherical_distortion_ext as ext
    from spherical_distortion import functional as F
    from spherical_distortion.nn import InterpolationType
    ext.clear_plan_cache()
    g = torch.Generator().manual_seed(81)
    with torch.inference_mode():
        x = torch.randn(2, 3, 16, 24, generator=g).cuda()
        m = (torch.rand(16, 24, 2, generator=g) * torch.tensor([31.0, 19.0])).cuda()
        a = F.resample(x, m, (20, 32), InterpolationType.BILINEAR)           # builds and caches a plan
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            b = F.resample(x, m, (20, 32), InterpolationType.BILINEAR)       # cache hit from another stream
        torch.cuda.current_stream().wait_stream(side)
        assert ext.plan_cache_size() == 1
        assert torch.equal(a, b)
        torch.testing.assert_close(a.cpu(), port.resample_to_map(x.cpu(), m.cpu(), 20, 32, 1), rtol=1e-5, atol=1e-5)
