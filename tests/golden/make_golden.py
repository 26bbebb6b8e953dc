"""Generate the golden fixtures of tests/golden/ from the reference itself.

Run in a container that has the reference checkout ($SPHERICAL_PACKAGE_REFERENCE,
else the folder `reference` beside this repository, or --reference PATH) and the
compiled reference CPU modules (python oracle/build_ref.py):

    python tests/golden/make_golden.py

Two files are written next to this script:

reference_kats.pt
    The known-answer vectors of the reference's own test suite
    (tests/test_mapped_convolution.py, test_mapped_transposed_convolution.py,
    test_mapped_pooling.py, test_resample.py; the *_cpu functions).  The test
    functions are executed unmodified against recording stand-ins for the layer
    classes and for tests/utils.py, so the inputs (tests/parameters.py) and the
    hand-computed expected outputs are captured as data.  Each case also stores
    what the reference's compiled CPU modules return for it (forward output and
    the gradients for an all-ones upstream gradient), after checking that the
    forward output equals the hand-computed vector.

reference_siblings.pt
    Seeded random cases of the operators beside the path that share its kernels: mapped average pooling and its
    backward (plain and weighted), UV-map gather / scatter and voting resampling, evaluated with the reference's
    compiled CPU modules; and the equirectangular kernel maps (grid, inverse gnomonic, inverse equirectangular) as
    the reference's own Python builders (layers/util/mapping_functions.py) return them in float32 and float64.

reference_random.pt
    Seeded random cases for everything the reference's tests do not pin
    (nearest / bispherical conv and pooling, every weighted op, float32, index
    contents, resample_to_map values, half-integer and out-of-range
    coordinates), evaluated with the reference's compiled CPU modules.
"""
import argparse
import importlib
import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import ref  # noqa: E402
from oracle.build_ref import default_reference  # noqa: E402


# --------------------------------------------------------------------------
# Part 1: harvest the reference's known-answer tests
# --------------------------------------------------------------------------
class _Layer:
    def __init__(self, kind, *a, **kw):
        self.kind, self.args, self.kwargs = kind, a, kw

    def double(self):
        return self


def _layer_cls(kind):
    return lambda *a, **kw: _Layer(kind, *a, **kw)


_current = {}


def _rec(**kw):
    _current.clear()
    _current.update(kw)
    return "OUTPUT", 0.0, 0.0, True


def harvest(reference):
    tests_dir = os.path.join(reference, "tests")
    sys.path.insert(0, tests_dir)
    params = importlib.import_module("parameters")
    enums = ref.mod("_enums")

    nn = types.ModuleType("spherical_distortion.nn")
    for n in ("MappedConvolution", "MappedTransposedConvolution", "MappedMaxPool", "MappedAvgPool",
              "Unresample", "Resample"):
        setattr(nn, n, _layer_cls(n))
    nn.InterpolationType = enums.InterpolationType
    pkg = types.ModuleType("spherical_distortion")
    pkg.nn = nn
    sys.modules["spherical_distortion"] = pkg
    sys.modules["spherical_distortion.nn"] = nn

    utils = types.ModuleType("utils")
    utils.mapped_conv_test = lambda layer, weight, input, sample_map, interp_weights=None, cuda=False: _rec(
        op="conv", layer=layer, weight=weight, input=input, sample_map=sample_map, interp_weights=interp_weights,
        bias=params.bias(weight.shape[0]))
    utils.mapped_transposed_conv_test = lambda layer, weight, input, oh, ow, sample_map, interp_weights=None, cuda=False: _rec(
        op="tconv", layer=layer, weight=weight, input=input, oh=oh, ow=ow, sample_map=sample_map,
        interp_weights=interp_weights, bias=params.bias(weight.shape[1]))
    utils.mapped_pool_test = lambda layer, input, sample_map, interp_weights=None, cuda=False: _rec(
        op="pool", layer=layer, input=input, sample_map=sample_map, interp_weights=interp_weights)
    utils.mapped_resample_test = lambda layer, input, sample_map, interp_weights=None, cuda=False: _rec(
        op="resample", layer=layer, input=input, sample_map=sample_map, interp_weights=interp_weights)
    sys.modules["utils"] = utils

    expected = {}

    def fake_allclose(out, correct, *a, **kw):
        assert out == "OUTPUT"
        expected["v"] = correct

    cases = []
    for fname in ("test_mapped_convolution", "test_mapped_transposed_convolution", "test_mapped_pooling",
                  "test_resample"):
        m = importlib.import_module(fname)
        m.testing = types.SimpleNamespace(assert_allclose=fake_allclose)
        for tname in [n for n in dir(m) if n.startswith("test_") and n.endswith("_cpu")]:
            _current.clear()
            expected.clear()
            getattr(m, tname)()
            c = dict(_current)
            layer = c.pop("layer")
            if layer.kind == "MappedAvgPool":
                continue  # average pooling is outside the path
            c["name"] = fname + "::" + tname
            c["layer_kind"] = layer.kind
            kw = dict(layer.kwargs)
            if layer.kind in ("Unresample", "Resample"):
                interp = layer.args[0] if layer.args else kw.get("interpolation", enums.InterpolationType.BILINEAR)
            else:
                interp = kw.get("interpolation", enums.InterpolationType.BILINEAR)
            c["interp"] = int(interp)
            c["kernel_size"] = kw.get("kernel_size")
            c["expected"] = expected["v"].clone()
            for k, v in list(c.items()):
                if torch.is_tensor(v):
                    c[k] = v.detach().clone()
            cases.append(c)
    return cases


def evaluate(c):
    """Run one harvested case through the reference's compiled CPU modules."""
    x, m, iw, it = c["input"], c["sample_map"].to(c["input"].dtype), c.get("interp_weights"), c["interp"]
    if iw is not None:
        iw = iw.to(x.dtype)
    c["sample_map"], c["interp_weights"] = m, iw
    if c["op"] == "conv":
        out = ref.mapped_conv_forward(x, m, c["weight"], c["bias"], c["kernel_size"], it, iw)
        g = ref.mapped_conv_backward(torch.ones_like(out), m, x, c["weight"], c["bias"], c["kernel_size"], it, iw)
        c["ref_grads"] = [t.clone() for t in g]
    elif c["op"] == "tconv":
        out = ref.mapped_transposed_conv_forward(x, m, c["weight"], c["bias"], c["oh"], c["ow"], c["kernel_size"], it, iw)
        g = ref.mapped_transposed_conv_backward(torch.ones_like(out), m, x, c["weight"], c["bias"],
                                                c["kernel_size"], it, iw)
        c["ref_grads"] = [t.clone() for t in g]
    elif c["op"] == "pool":
        out, idx = ref.mapped_max_pool(x, m, c["kernel_size"], it, iw)
        c["ref_idx"] = idx.clone()
        c["ref_grads"] = [ref.mapped_max_unpool(torch.ones_like(out), idx, m, x.shape[2], x.shape[3],
                                                c["kernel_size"], it, iw).clone()]
    else:
        out = ref.resample_from_map(x, m, it, iw)
        c["ref_grads"] = [ref.resample_to_map(torch.ones_like(out), m, x.shape[2], x.shape[3], it, iw).clone()]
    c["ref_output"] = out.clone()
    # the hand-computed vector broadcasts over batch and channels
    assert torch.allclose(out, c["expected"].to(out.dtype).expand_as(out), rtol=1e-7, atol=1e-9), c["name"]
    return c


# --------------------------------------------------------------------------
# Part 2: seeded random cases for what the reference's tests leave unpinned
# --------------------------------------------------------------------------
def _coords(g, shape, W, H, dtype):
    """Coordinates that cover interior, half-integer ties and out-of-range."""
    m = torch.rand(*shape, 2, generator=g, dtype=torch.float64)
    m[..., 0] = m[..., 0] * (W + 3) - 1.5
    m[..., 1] = m[..., 1] * (H + 3) - 1.5
    flat = m.view(-1, 2)
    n = flat.shape[0]
    ties = torch.randperm(n, generator=g)[: max(1, n // 6)]
    flat[ties] = torch.floor(flat[ties]) + 0.5           # exact .5 ties for llround
    ints = torch.randperm(n, generator=g)[: max(1, n // 6)]
    flat[ints] = torch.floor(flat[ints])                 # exact integers
    return m.to(dtype)


def random_cases():
    cases = []
    seed = 1000
    for dtype in (torch.float64, torch.float32):
        for interp in (0, 1, 2):
            for P in (0, 3):
                seed += 1
                g = torch.Generator().manual_seed(seed)
                B, Cin, Cout, IH, IW, OH, OW, K = 2, 3, 4, 6, 9, 5, 7, 4
                x = torch.randn(B, Cin, IH, IW, generator=g, dtype=dtype)
                shape = (OH, OW, K, P) if P else (OH, OW, K)
                m = _coords(g, shape, IW, IH, dtype)
                iw = torch.rand(OH, OW, K, P, generator=g, dtype=dtype) if P else None
                w = torch.randn(Cout, Cin, K, generator=g, dtype=dtype)
                b = torch.randn(Cout, generator=g, dtype=dtype)
                go = torch.randn(B, Cout, OH, OW, generator=g, dtype=dtype)
                c = dict(op="conv", seed=seed, interp=interp, kernel_size=K, input=x, sample_map=m,
                         interp_weights=iw, weight=w, bias=b, grad_output=go)
                c["ref_output"] = ref.mapped_conv_forward(x, m, w, b, K, interp, iw)
                c["ref_grads"] = list(ref.mapped_conv_backward(go, m, x, w, b, K, interp, iw))
                cases.append(c)

                # transposed conv: map has the input's size and points into the (IH, IW) output grid
                xt = torch.randn(B, Cout, OH, OW, generator=g, dtype=dtype)
                wt = torch.randn(Cout, Cin, K, generator=g, dtype=dtype)   # (in=Cout, out=Cin, K)
                bt = torch.randn(Cin, generator=g, dtype=dtype)
                got = torch.randn(B, Cin, IH, IW, generator=g, dtype=dtype)
                c = dict(op="tconv", seed=seed, interp=interp, kernel_size=K, input=xt, sample_map=m,
                         interp_weights=iw, weight=wt, bias=bt, oh=IH, ow=IW, grad_output=got)
                c["ref_output"] = ref.mapped_transposed_conv_forward(xt, m, wt, bt, IH, IW, K, interp, iw)
                c["ref_grads"] = list(ref.mapped_transposed_conv_backward(got, m, xt, wt, bt, K, interp, iw))
                cases.append(c)

                # max pool on strictly positive input (so the reference's CPU sentinel never triggers)
                xp = torch.rand(B, Cin, IH, IW, generator=g, dtype=dtype) + 0.5
                mp = m.clone()
                mp[..., 0] = mp[..., 0].clamp(0, IW - 1)   # every sample inside: values stay positive
                mp[..., 1] = mp[..., 1].clamp(0, IH - 1)
                out, idx = ref.mapped_max_pool(xp, mp, K, interp, iw)
                gp = torch.randn(B, Cin, OH, OW, generator=g, dtype=dtype)
                c = dict(op="pool", seed=seed, interp=interp, kernel_size=K, input=xp, sample_map=mp,
                         interp_weights=iw, grad_output=gp, ref_output=out, ref_idx=idx)
                c["ref_grads"] = [ref.mapped_max_unpool(gp, idx, mp, IH, IW, K, interp, iw)]
                cases.append(c)

                # resample_from_map / resample_to_map
                rm = m[:, :, 0].contiguous()
                riw = iw[:, :, 0].contiguous() if P else None
                y = torch.randn(B, Cin, OH, OW, generator=g, dtype=dtype)
                c = dict(op="resample", seed=seed, interp=interp, input=x, sample_map=rm, interp_weights=riw,
                         grad_output=y)
                c["ref_output"] = ref.resample_from_map(x, rm, interp, riw)
                c["ref_grads"] = [ref.resample_to_map(y, rm, IH, IW, interp, riw)]
                cases.append(c)
    # max pool with negative inputs: pins the reference CPU's sentinel behaviour (idx = -1 rows)
    g = torch.Generator().manual_seed(77)
    xn = torch.randn(2, 3, 6, 9, generator=g, dtype=torch.float32)
    mn = _coords(g, (5, 7, 2), 9, 6, torch.float32)
    out, idx = ref.mapped_max_pool(xn, mn, 2, 0, None)
    cases.append(dict(op="pool_sentinel", seed=77, interp=0, kernel_size=2, input=xn, sample_map=mn,
                      interp_weights=None, ref_output=out, ref_idx=idx))
    for c in cases:
        for k, v in list(c.items()):
            if torch.is_tensor(v):
                c[k] = v.detach().clone()
            elif isinstance(v, list):
                c[k] = [t.detach().clone() for t in v]
    return cases


# --------------------------------------------------------------------------
# Part 3: sibling operators and kernel maps
# --------------------------------------------------------------------------
def sibling_cases(reference):
    cases = []
    seed = 2000
    for dtype in (torch.float64, torch.float32):
        for interp in (0, 1, 2):
            for P in (0, 3):
                seed += 1
                g = torch.Generator().manual_seed(seed)
                B, C, IH, IW, OH, OW, K = 2, 3, 6, 9, 5, 7, 4
                x = torch.randn(B, C, IH, IW, generator=g, dtype=dtype)
                shape = (OH, OW, K, P) if P else (OH, OW, K)
                m = _coords(g, shape, IW, IH, dtype)
                iw = torch.rand(OH, OW, K, P, generator=g, dtype=dtype) if P else None
                gp = torch.randn(B, C, OH, OW, generator=g, dtype=dtype)
                cases.append(dict(op="avgpool", seed=seed, interp=interp, kernel_size=K, input=x, sample_map=m,
                                  interp_weights=iw, grad_output=gp,
                                  ref_output=ref.mapped_avg_pool(x, m, K, interp, iw),
                                  ref_grads=[ref.mapped_avg_unpool(gp, m, IH, IW, K, interp, iw)]))
            # UV maps: 5 textures of 6 x 7 texels gathered into / scattered from an 8 x 11 image
            seed += 1
            g = torch.Generator().manual_seed(seed)
            B, C, NT, TH, TW, IH, IW = 2, 3, 5, 6, 7, 8, 11
            tex = torch.randn(B, C, NT, TH, TW, generator=g, dtype=dtype)
            quad = torch.randint(0, NT, (IH, IW), generator=g)
            uv = _coords(g, (IH, IW), TW, TH, dtype)
            img = torch.randn(B, C, IH, IW, generator=g, dtype=dtype)
            cases.append(dict(op="uv", seed=seed, interp=interp, input=tex, quad_idx=quad, tex_uv=uv, grad_output=img,
                              ref_output=ref.resample_from_uv_maps(tex, quad, uv, interp),
                              ref_grads=[ref.resample_to_uv_maps(img, quad, uv, NT, TH, TW, interp)]))
    for seed, (IH, IW, OH, OW, NC) in ((2101, (12, 16, 5, 7, 6)), (2102, (6, 6, 9, 9, 3)), (2103, (20, 24, 2, 3, 11))):
        g = torch.Generator().manual_seed(seed)
        # one channel: with more, the reference's vote tensor overlaps channels (it steps the channel by OH*OW instead
        # of OH*OW*num_candidates, ext_modules/include/common/resample.h:127-129), which pins nothing useful
        lab = torch.randint(0, NC, (2, 1, IH, IW), generator=g)
        m = torch.stack((torch.randint(-1, OW + 1, (IH, IW), generator=g), torch.randint(-1, OH + 1, (IH, IW), generator=g)), -1)
        cases.append(dict(op="voting", seed=seed, input=lab, sample_map=m, oh=OH, ow=OW, num_candidates=NC,
                          ref_output=ref.voting_resample_to_map(lab, m, OH, OW, NC)))
    # kernel maps from the reference's own Python builders (its package is mounted unmodified on this repo's extension)
    sys.path.insert(0, os.path.join(ROOT, "spherical-package_b200"))
    from _spherical_distortion_ext import reference_compat as rc
    rc.install_placeholders()
    rc.mount_reference_layers(os.path.join(reference, "layers"))
    import spherical_distortion.util as u
    for kind, fn in (("grid", u.grid_projection_map), ("inverse_gnomonic", u.inverse_gnomonic_projection_map),
                     ("inverse_equirectangular", u.inverse_equirectangular_projection_map)):
        for (H, W, kh, kw, stride, dil) in ((8, 16, 3, 3, 1, 1), (12, 20, 3, 3, 2, 1), (7, 10, 5, 3, 1, 2), (9, 14, 2, 2, 3, 1)):
            c = dict(op="map", kind=kind, H=H, W=W, kh=kh, kw=kw, stride=stride, dilation=dil)
            for name, dt in (("f32", torch.float32), ("f64", torch.float64)):
                old = torch.get_default_dtype()
                torch.set_default_dtype(dt)
                try:
                    c[name] = fn((H, W), (kh, kw), stride, dil).clone()
                finally:
                    torch.set_default_dtype(old)
            cases.append(c)
    for c in cases:
        for k, v in list(c.items()):
            if torch.is_tensor(v):
                c[k] = v.detach().clone()
            elif isinstance(v, list):
                c[k] = [t.detach().clone() for t in v]
    return cases


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference())
    ap.add_argument("--only", nargs="+", default=["kats", "random", "siblings"], choices=["kats", "random", "siblings"],
                    help="which fixture files to (re)write; the reference's scatters add with OpenMP atomics, so a rewritten "
                         "file differs from the committed one in the last bit of some gradients")
    a = ap.parse_args()
    assert ref.available(), "build the reference modules first: python oracle/build_ref.py"
    if "kats" in a.only:
        kats = [evaluate(c) for c in harvest(a.reference)]
        torch.save(kats, os.path.join(HERE, "reference_kats.pt"))
        print("reference_kats.pt: %d cases" % len(kats))
        for c in kats:
            print("  ", c["name"], c["op"], "interp", c["interp"], tuple(c["input"].shape))
    if "random" in a.only:
        rnd = random_cases()
        torch.save(rnd, os.path.join(HERE, "reference_random.pt"))
        print("reference_random.pt: %d cases" % len(rnd))
    if "siblings" in a.only:
        sib = sibling_cases(a.reference)
        torch.save(sib, os.path.join(HERE, "reference_siblings.pt"))
        print("reference_siblings.pt: %d cases" % len(sib))
