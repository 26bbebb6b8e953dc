"""CPU-only checks of the boundary: the C-ABI library loads and exports every symbol the header declares, the
host-side size queries work without a GPU, and the plugin package exposes the reference's module/function names."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "sphmap.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sph_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from sphmap import capi
    declared = _declared_symbols()
    assert len(declared) >= 22
    for name in declared:
        assert hasattr(capi.lib, name), name
    assert sorted(capi.SYMBOLS) == declared


def test_host_side_queries_need_no_gpu():
    from sphmap import capi
    assert capi.lib.sph_version() >= 100
    assert capi.lib.sph_status_string(0) == b"ok"
    n = capi.lib.sph_plan_bytes(*capi._ints(20, 4, 0), 1, *capi._ints(4, 5), 0)
    assert n > 0 and n % 256 == 0
    assert capi.lib.sph_plan_bytes(*capi._ints(0, 4, 0), 1, *capi._ints(4, 5), 0) == 0          # empty map
    assert capi.lib.sph_plan_bytes(*capi._ints(1 << 40, 4, 0), 1, *capi._ints(4, 5), 0) == 0    # too large
    # exact path: only the weight-gradient op needs scratch
    q = lambda op, prec: capi.lib.sph_conv_workspace_bytes(op, *capi._ints(2, 16, 32, 64, 128, 64, 128, 9, 0), 0, 1, prec)  # noqa: E731
    assert q(capi.CONV_FORWARD, capi.EXACT) == 0 and q(capi.CONV_BACKWARD_WEIGHT, capi.EXACT) > 0
    assert q(capi.CONV_FORWARD, capi.BF16) > 0
    assert capi.lib.sph_conv_workspace_bytes(0, *capi._ints(2, 16, 32, 64, 128, 64, 128, 9, 0), 1, 1, capi.BF16) == 0  # f64+bf16


def test_invalid_arguments_are_rejected_before_any_launch():
    from sphmap import capi
    null = ctypes.c_void_p(0)
    rc = capi.lib.sph_resample_from_map(null, null, null, null, *capi._ints(1, 1, 4, 4, 2, 2, 0), 0, 1, null)
    assert rc == 1 and b"invalid" in capi.lib.sph_status_string(rc)
    rc = capi.lib.sph_mapped_conv_forward(null, null, null, null, null, null, *capi._ints(1, 1, 1, 4, 4, 2, 2, 1, 0), 7, 1, 0,
                                          null, ctypes.c_size_t(0), null)
    assert rc == 2   # unsupported dtype


def test_plugin_package_has_the_reference_module_and_function_names():
    import importlib
    expect = {
        "_enums": ["InterpolationType", "DistortionType"],
        "_resample": ["resample_to_map", "resample_from_map"],
        "_weighted_resample": ["weighted_resample_to_map", "weighted_resample_from_map"],
        "_mapped_max_pooling": ["mapped_max_pool", "mapped_max_unpool"],
        "_weighted_mapped_max_pooling": ["weighted_mapped_max_pool", "weighted_mapped_max_unpool"],
        "_mapped_convolution": ["mapped_conv_forward", "mapped_conv_backward"],
        "_weighted_mapped_convolution": ["weighted_mapped_conv_forward", "weighted_mapped_conv_backward"],
        "_mapped_transposed_convolution": ["mapped_transposed_conv_forward", "mapped_transposed_conv_backward"],
        "_weighted_mapped_transposed_convolution": ["weighted_mapped_transposed_conv_forward",
                                                    "weighted_mapped_transposed_conv_backward"],
        # modules beside the path that the reference's Python layer imports unconditionally
        "_mapped_avg_pooling": ["mapped_avg_pool", "mapped_avg_unpool"],
        "_weighted_mapped_avg_pooling": ["weighted_mapped_avg_pool", "weighted_mapped_avg_unpool"],
        "_uv_resample": ["resample_to_uv_maps", "resample_from_uv_maps"],
        "_voting_resample": ["voting_resample_to_map"],
        "_convolution": ["conv_forward", "conv_backward"],
        "_transposed_convolution": ["transposed_conv_forward", "transposed_conv_backward"],
        "_distort": ["create_distortion_sample_map", "DistortionType"],
    }
    for mod, names in expect.items():
        m = importlib.import_module("_spherical_distortion_ext." + mod)
        for n in names:
            assert hasattr(m, n), (mod, n)
    from _spherical_distortion_ext._enums import InterpolationType as I
    assert [int(I.NEAREST), int(I.BILINEAR), int(I.BISPHERICAL)] == [0, 1, 2]
    assert I(torch.tensor(2)) == I.BISPHERICAL          # 0-d tensors round-trip like in the reference's backward


def test_plugin_refuses_cpu_tensors_and_checks_shapes():
    import _spherical_distortion_ext._mapped_convolution as mc
    from _spherical_distortion_ext._enums import InterpolationType as I
    x, m, w, b = torch.zeros(1, 2, 4, 4), torch.zeros(2, 2, 3, 2), torch.zeros(5, 2, 3), torch.zeros(5)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        mc.mapped_conv_forward(x, m, w, b, 3, I.BILINEAR)


def test_mirror_layer_assertions_match_the_reference():
    from spherical_distortion.nn import MappedConvolution, MappedMaxPool, Unresample
    layer = MappedConvolution(2, 3, 4)
    assert tuple(layer.weight.shape) == (3, 2, 4) and tuple(layer.bias.shape) == (3,)
    with pytest.raises(AssertionError, match="same dtype"):
        layer(torch.zeros(1, 2, 4, 5), torch.zeros(4, 5, 4, 2).double())
    with pytest.raises(AssertionError, match="Kernel size"):
        layer(torch.zeros(1, 2, 4, 5), torch.zeros(4, 5, 3, 2))
    with pytest.raises(AssertionError, match="4 dimensions"):
        MappedMaxPool(4)(torch.zeros(2, 4, 5), torch.zeros(4, 5, 4, 2))
    with pytest.raises(AssertionError, match="3 or 4"):
        Unresample()(torch.zeros(4, 5), torch.zeros(4, 5, 2))


def test_workload_generators_have_the_configured_shapes():
    from sphmap import workloads as wl
    c0 = wl.config0()
    assert tuple(c0["map"].shape) == (64, 128, 9, 2) and c0["map"][..., 0].min() >= 0 and c0["map"][..., 0].max() < 128
    assert tuple(wl.tangent_image_map(512, 1024).shape) == (1280, 64, 2)
    assert wl.icosahedron_face_centres().shape == (20, 2)
    assert abs(wl.encoder_flops(64) / 1e9 - 4049.08) < 0.01
    c4 = wl.config4(B=1, H=64, W=128)
    assert [tuple(m.shape[:2]) for m in c4["maps"]] == [(32, 64), (16, 32), (16, 32), (16, 32)]


def test_reference_python_layer_imports_unmodified_on_this_package():
    """The reference's own `layers/` folder, mounted as `spherical_distortion` without a change, imports completely on
    top of this package: every native module name it asks for resolves (the mesh / lens-distortion modules and the
    absent third-party packages through import-time stand-ins).  Needs the reference checkout
    ($SPHERICAL_PACKAGE_REFERENCE or a folder `reference` beside the repository); run in a child process so that the
    mirror package of the same name, which other tests import, is not disturbed."""
    import subprocess
    import sys
    from oracle.build_ref import default_reference
    layers = os.path.join(default_reference(), "layers")
    if not os.path.isdir(layers):
        pytest.skip("reference checkout not present")
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "from _spherical_distortion_ext import reference_compat as rc\n"
        "rc.install_placeholders(); rc.mount_reference_layers(%r)\n"
        "import spherical_distortion.nn as nn, spherical_distortion.functional as F, spherical_distortion.util as u\n"
        "assert nn.__file__.startswith(%r)\n"
        "for n in ('MappedConvolution','MappedTransposedConvolution','MappedMaxPool','MappedAvgPool','Resample','Unresample','ResampleFromUV','Convolution'): getattr(nn, n)\n"
        "for n in ('mapped_convolution','mapped_max_pool','mapped_avg_pool','resample','unresample','uv_resample','voting_resample','convolution'): getattr(F, n)\n"
        "print('imported', tuple(u.inverse_gnomonic_projection_map((8, 16), (3, 3)).shape))\n"
    ) % (os.path.join(ROOT, "spherical-package_b200"), layers, layers)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    assert "imported (8, 16, 9, 2)" in r.stdout
