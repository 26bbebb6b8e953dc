"""Failure detection of the tensor-core kernels without faulting anything: every device-side wait is bounded, a wait
that runs out is reported through a status word, and the context stays usable.  The library's own self check makes
such a wait run out on purpose (an mbarrier nothing arrives at, 1 ms limit); nothing here traps, hangs or touches a
bad address."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_reports_status_and_leaves_the_device_usable():
    from sphmap import capi
    from oracle import port
    capi.device_status(reset=True)
    assert capi.device_status(reset=False) == 0
    assert capi.debug_bounded_wait(limit_ns=1_000_000) == 1          # the kernel returned and said so
    assert capi.device_status(reset=False) == 1                     # sticky word set ...
    with pytest.raises(capi.SphError):
        capi.check_device_status()                                  # ... raises, and clears
    assert capi.device_status() == 0
    # tensor memory was freed and the context is intact: a tensor-core convolution runs and is right
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, 64, 16, 32, generator=g)
    w = torch.randn(64, 64, 9, generator=g) / 24.0
    b = torch.zeros(64)
    m = torch.rand(16, 32, 9, 2, generator=g) * torch.tensor([32.0, 16.0])
    ws = capi.conv_workspace(capi.CONV_FORWARD, 1, 64, 64, 16, 32, 16, 32, 9, 0, capi.F32, 1, capi.BF16, x.cuda())
    out = capi.conv_forward(x.cuda(), m.cuda(), w.cuda(), b.cuda(), 9, 1, None, capi.BF16, ws=ws)
    ref = port.mapped_conv_forward(x, m, w, b, 9, 1)
    assert (out.cpu() - ref).abs().max() <= 2e-2 * ref.abs().max()
    assert capi.workspace_status(ws) == 0 and capi.device_status() == 0


def test_plugin_reports_device_status():
    import _spherical_distortion_ext as ext
    from sphmap import capi
    assert ext.device_status() == 0
    assert capi.debug_bounded_wait(limit_ns=200_000) == 1
    assert ext.device_status() == 1 and ext.device_status() == 0
