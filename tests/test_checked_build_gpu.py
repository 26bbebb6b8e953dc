"""The bounds-checked build of the library (libsphmap_checked.so, -DSPH_BOUNDS_CHECK), the stand-in for a memory
checker: the reference's known-answer cases and small random maps with out-of-range, infinite and NaN coordinates
run through it in a child process; every result must still match the oracle and the status word must stay clear,
i.e. no kernel tried to use an index outside its range.  Also in every build: a plan made for tensors of another
size is refused by its header (the operator writes zeros) instead of being followed."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys
sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "spherical-package_b200")); sys.path.insert(0, os.path.join(ROOT, "tests"))
import torch
from sphmap import capi
from oracle import port
from _gpu_impl import CApi
assert capi.lib.sph_build_is_checked() == 1, "the checked library was not loaded"
assert capi.device_status() == 0

def close(a, b, tol=1e-5):
    t = tol if b.dtype == torch.float32 else 1e-11
    torch.testing.assert_close(a, b, rtol=t, atol=t * max(1.0, b.abs().max().item()))

impl = CApi()
n = 0
for c in torch.load(os.path.join(ROOT, "tests", "golden", "reference_kats.pt"), weights_only=False):
    x, m, iw, it, K = c["input"], c["sample_map"], c.get("interp_weights"), c["interp"], c.get("kernel_size")
    if c["op"] == "conv":
        close(impl.mapped_conv_forward(x, m, c["weight"], c["bias"], K, it, iw), c["ref_output"])
        for a, b in zip(impl.mapped_conv_backward(torch.ones_like(c["ref_output"]), m, x, c["weight"], c["bias"], K, it, iw), c["ref_grads"]):
            close(a, b)
    elif c["op"] == "tconv":
        close(impl.mapped_transposed_conv_forward(x, m, c["weight"], c["bias"], c["oh"], c["ow"], K, it, iw), c["ref_output"])
        for a, b in zip(impl.mapped_transposed_conv_backward(torch.ones_like(c["ref_output"]), m, x, c["weight"], c["bias"], K, it, iw), c["ref_grads"]):
            close(a, b)
    elif c["op"] == "pool":
        out, idx = impl.mapped_max_pool(x, m, K, it, iw)
        assert torch.equal(out, c["ref_output"]) and torch.equal(idx, c["ref_idx"])
        close(impl.mapped_max_unpool(torch.ones_like(out), idx, m, x.shape[2], x.shape[3], K, it, iw), c["ref_grads"][0])
    else:
        assert torch.equal(impl.resample_from_map(x, m, it, iw), c["ref_output"])
        close(impl.resample_to_map(torch.ones_like(c["ref_output"]), m, x.shape[2], x.shape[3], it, iw), c["ref_grads"][0])
    n += 1
assert n == 23 and capi.device_status() == 0, "known-answer cases"

# random small maps with hostile coordinates: far out of range, +-inf, NaN, exact half-integers
g = torch.Generator().manual_seed(123)
for dtype in (torch.float32, torch.float64):
    for interp in (0, 1, 2):
        for P in (0, 2):
            B, C, IH, IW, OH, OW, K = 2, 3, 8, 16, 8, 16, 4
            x = torch.randn(B, C, IH, IW, generator=g, dtype=dtype)
            shape = (OH, OW, K, P, 2) if P else (OH, OW, K, 2)
            m = (torch.rand(*shape, generator=g, dtype=torch.float64) * torch.tensor([IW + 8.0, IH + 8.0]) - 4.0).to(dtype)
            flat = m.view(-1, 2)
            flat[0] = float("nan"); flat[1, 0] = float("inf"); flat[2, 1] = -float("inf"); flat[3] = 1e30; flat[4] = -1e30
            flat[5] = torch.tensor([2.5, 3.5], dtype=dtype); flat[6] = torch.tensor([-0.5, IH - 0.5], dtype=dtype)
            iw = torch.rand(OH, OW, K, P, generator=g, dtype=dtype) if P else None
            w = torch.randn(5, C, K, generator=g, dtype=dtype); b = torch.randn(5, generator=g, dtype=dtype)
            go = torch.randn(B, 5, OH, OW, generator=g, dtype=dtype)
            xd, md, iwd, wd, bd, god = [None if t is None else t.cuda() for t in (x, m, iw, w, b, go)]
            outs = []
            outs.append(capi.conv_forward(xd, md, wd, bd, K, interp, iwd))
            plan = capi.plan_build(md, iwd, OH * OW, K, interp, IH, IW)
            outs.append(capi.conv_backward_input(god, plan, wd, IH, IW, K))
            outs += list(capi.conv_backward_weight(god, xd, md, K, interp, iwd))
            po, idx = capi.mapped_max_pool(xd, md, K, interp, iwd)
            gp = torch.randn(B, C, OH, OW, generator=g, dtype=dtype).cuda()
            outs += [po, capi.mapped_max_unpool(gp, idx, md, IH, IW, K, interp, iwd),
                     capi.mapped_max_unpool_planned(gp, idx, capi.slot_plan_build(md, iwd, K, interp, IH, IW), IH, IW, K, P),
                     capi.mapped_avg_pool(xd, md, K, interp, iwd),
                     capi.mapped_avg_unpool(gp, capi.slot_plan_build(md, iwd, K, interp, IH, IW), IH, IW, K)]
            rm, riw = md[:, :, 0].contiguous(), (None if iwd is None else iwd[:, :, 0].contiguous())
            outs.append(capi.resample_from_map(xd, rm, interp, riw))
            rplan = capi.plan_build(rm, riw, OH * OW, 1, interp, IH, IW)
            outs += [capi.resample_to_map(gp, rplan, IH, IW), capi.resample_to_map_normalized(gp, rplan, IH, IW)]
            if dtype == torch.float32 and P == 0:      # tensor-core kernels on the same hostile map
                x64 = torch.randn(B, 64, IH, IW, generator=g).cuda(); w64 = (torch.randn(64, 64, K, generator=g) / 16).cuda()
                b64 = torch.zeros(64).cuda(); g64 = torch.randn(B, 64, OH, OW, generator=g).cuda()
                outs.append(capi.conv_forward(x64, md, w64, b64, K, interp, None, capi.BF16))
                outs.append(capi.conv_backward_input(g64, plan, w64, IH, IW, K, capi.BF16))
                outs += list(capi.conv_backward_weight(g64, x64, md, K, interp, None, capi.BF16))
                # and the large-tile exact float32 kernels (64 output rows, 64 gathered channels)
                e_out = capi.conv_forward(x64, md, w64, b64, K, interp, None)
                outs += [e_out, capi.conv_backward_input(g64, plan, w64, IH, IW, K)]
                outs += list(capi.conv_backward_weight(g64, x64, md, K, interp, None))
                mm64 = m.clone(); mm64.view(-1, 2)[:5] = -100.0
                close(e_out.cpu(), port.mapped_conv_forward(x64.cpu(), mm64, w64.cpu(), b64.cpu(), K, interp, None), 1e-4)
            if dtype == torch.float32:                 # the thin layer's own tensor-core kernels (3 channels, bf16 precision)
                w16 = (torch.randn(16, C, K, generator=g) / 3).cuda(); b16 = torch.zeros(16).cuda()
                g16 = torch.randn(B, 16, OH, OW, generator=g).cuda()
                outs.append(capi.conv_forward(xd, md, w16, b16, K, interp, iwd, capi.BF16))
                outs.append(capi.conv_backward_input(g16, plan, w16, IH, IW, K, capi.BF16))
                outs += list(capi.conv_backward_weight(g16, xd, md, K, interp, iwd, capi.BF16))
            for t in outs:
                assert torch.isfinite(t).all(), (dtype, interp, P)
            # NaN, infinite and astronomically large coordinates have no tap in this library (the reference converts
            # them to integers with undefined behaviour); the oracle gets a plainly outside point in their place
            mm = m.clone(); mm.view(-1, 2)[:5] = -100.0
            close(outs[0].cpu(), port.mapped_conv_forward(x, mm, w, b, K, interp, iw), 1e-4)
            close(outs[9].cpu(), port.resample_from_map(x, mm[:, :, 0].contiguous(), interp, None if iw is None else iw[:, :, 0].contiguous()), 1e-6)
            assert capi.device_status() == 0, ("index out of range", dtype, interp, P)
print("checked-build cases ok")
'''


def test_checked_build_sees_no_out_of_range_index():
    lib = os.path.join(ROOT, "spherical-package_b200", "_spherical_distortion_ext", "libsphmap_checked.so")
    assert os.path.exists(lib), "libsphmap_checked.so has not been built (python build.py --checked)"
    env = dict(os.environ, SPHMAP_LIBRARY="checked")
    r = subprocess.run([sys.executable, "-c", "ROOT = %r\n" % ROOT + CHILD], capture_output=True, text=True, env=env, timeout=900)
    assert r.returncode == 0 and "checked-build cases ok" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])


def test_plan_made_for_another_size_is_refused_not_followed():
    from sphmap import capi
    assert capi.lib.sph_build_is_checked() == 0
    g = torch.Generator().manual_seed(9)
    m_small = (torch.rand(8, 8, 2, generator=g) * 16).cuda()
    plan_small = capi.plan_build(m_small, None, 64, 1, 1, 16, 16)          # made for an 8 x 8 source
    x_big = torch.randn(1, 2, 32, 32, generator=g).cuda()                  # a 32 x 32 source is passed
    out = capi.resample_to_map(x_big, plan_small, 16, 16)
    assert torch.count_nonzero(out) == 0
    assert capi.device_status() == 0
