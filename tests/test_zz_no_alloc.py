"""The allocation-free resample_to_map entry point (collected last on purpose).

Some hosts of this library are not allowed to allocate device memory around a call: they run inside a memory
budget fixed at start-up, or in a loop where an allocation could stall, or they are handed pre-allocated buffers
only.  `sph_resample_to_map_static` serves them by keeping the scatter plan in an array inside the library.  Here
it is called through the C ABI twice in a row, with different maps and sizes so that whatever the first call left
in the shared array would show up in the second, and each result is compared with the ordinary entry point
(plan in caller scratch), which shares the kernels: the results must be identical.  One case is also compared
directly with the CPU oracle, and one is large enough to run the four-pixels-per-thread scatter kernel."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, B, C, MH, MW, OH, OW, P, interp, dtype):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, C, MH, MW, generator=g, dtype=dtype)
    shape = (MH, MW, P, 2) if P else (MH, MW, 2)
    m = (torch.rand(*shape, generator=g, dtype=torch.float64) * torch.tensor([OW + 2.0, OH + 2.0]) - 1.0).to(dtype)
    iw = torch.rand(MH, MW, P, generator=g, dtype=dtype) if P else None
    return [t.cuda() if t is not None else None for t in (x, m, iw)]


def test_static_scratch_entry_matches_the_regular_one_twice_in_a_row():
    from sphmap import capi
    before = torch.cuda.memory_allocated()
    cases = [(1, 3, 5, 40, 64, 33, 47, 0, 1, torch.float32), (2, 2, 4, 24, 31, 50, 70, 3, 2, torch.float64)]
    for seed, B, C, MH, MW, OH, OW, P, interp, dtype in cases:
        x, m, iw = _case(seed, B, C, MH, MW, OH, OW, P, interp, dtype)
        out = torch.full((B, C, OH, OW), float("nan"), dtype=dtype, device="cuda")
        held = torch.cuda.memory_allocated()
        capi.resample_to_map_static(x, m, OH, OW, interp, iw, out=out)
        assert torch.cuda.memory_allocated() == held          # the call itself took nothing from the allocator
        plan = capi.plan_build(m, iw, MH * MW, 1, interp, OH, OW)
        ref = capi.resample_to_map(x, plan, OH, OW)
        assert torch.equal(out, ref), (seed, (out - ref).abs().max().item())
        assert torch.isfinite(out).all()
        # and against the CPU oracle itself (adds in another order: 1e-5 relative to the tensor's scale)
        from oracle import port
        want = port.resample_to_map(x.cpu(), m.cpu(), OH, OW, interp, None if iw is None else iw.cpu())
        torch.testing.assert_close(out.cpu(), want, rtol=1e-5, atol=1e-5 * want.abs().max().item())
    del x, m, iw, out, plan, ref
    assert torch.cuda.memory_allocated() <= before + (1 << 20)


def test_static_scratch_entry_large_destination_selects_the_four_pixel_kernel():
    """Nearest map, 512x512 destination, 20 planes: the plan (2.6 MB) still fits the built-in array and the scatter
    runs on the kernel that writes four destination pixels per thread."""
    from sphmap import capi
    from oracle import port
    B, C, MH, MW, OH, OW = 4, 5, 256, 256, 512, 512
    assert capi.lib.sph_plan_bytes(*capi._ints(MH * MW, 1, 0), 0, *capi._ints(OH, OW), 0) <= capi.STATIC_SCRATCH_BYTES
    x, m, _ = _case(5, B, C, MH, MW, OH, OW, 0, 0, torch.float32)
    out = torch.full((B, C, OH, OW), float("nan"), device="cuda")
    for _ in range(2):
        capi.resample_to_map_static(x, m, OH, OW, 0, None, out=out)
    plan = capi.plan_build(m, None, MH * MW, 1, 0, OH, OW)
    assert torch.equal(out, capi.resample_to_map(x, plan, OH, OW))
    want = port.resample_to_map(x.cpu(), m.cpu(), OH, OW, 0)
    torch.testing.assert_close(out.cpu(), want, rtol=1e-5, atol=1e-5 * want.abs().max().item())


def test_static_scratch_entry_rejects_bad_sizes_before_touching_the_array():
    from sphmap import capi
    x, m, _ = _case(6, 1, 1, 8, 8, 8, 8, 0, 1, torch.float32)
    out = torch.zeros(1, 1, 8, 8, device="cuda")
    rc = capi.lib.sph_resample_to_map_static(capi._ptr(x), capi._ptr(m), None, capi._ptr(out), *capi._ints(-1, 1, 8, 8, 8, 8, 0),
                                             ctypes.c_int(0), ctypes.c_int(1), capi._stream())
    assert rc == 1


def test_static_scratch_entry_rejects_oversized_problems():
    from sphmap import capi
    # 2048 x 2048 destination: the offsets table alone exceeds the 8 MiB array
    n = capi.lib.sph_plan_bytes(*capi._ints(64 * 64, 1, 0), 1, *capi._ints(2048, 2048), 0)
    assert n > capi.STATIC_SCRATCH_BYTES
    x = torch.zeros(1, 1, 64, 64, device="cuda")
    m = torch.zeros(64, 64, 2, device="cuda")
    out = torch.zeros(1, 1, 8, 8, device="cuda")
    rc = capi.lib.sph_resample_to_map_static(capi._ptr(x), capi._ptr(m), None, capi._ptr(out), *capi._ints(1, 1, 64, 64, 2048, 2048, 0),
                                             ctypes.c_int(0), ctypes.c_int(1), capi._stream())
    assert rc == 6 and b"static" in capi.lib.sph_status_string(rc)
