"""The reference's own CPU modules (built by oracle/build_ref.py) behind the
same function signatures as oracle/port.py.

TEST INFRASTRUCTURE ONLY.  ``available()`` is False when ``oracle/_ref`` has not
been built (it needs the reference checkout at build time, not at run time).
The shared objects are loaded under a private package name so that they never
shadow the product's ``_spherical_distortion_ext``.
"""
import importlib.util
import os
import sysconfig

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "_spherical_distortion_ext")
_mods = {}


def _path(name):
    return os.path.join(_DIR, name + sysconfig.get_config_var("EXT_SUFFIX"))


def available():
    return os.path.exists(_path("_mapped_convolution")) and os.path.exists(_path("_enums"))


def mod(name):
    """Load one compiled reference module (e.g. '_resample')."""
    if name not in _mods:
        import torch  # noqa: F401  (libtorch must be loaded first)
        spec = importlib.util.spec_from_file_location(name, _path(name))
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        _mods[name] = m
    return _mods[name]


def interp_enum(interp):
    return mod("_enums").InterpolationType(int(interp))


def _c(*ts):
    return [None if t is None else t.detach().contiguous() for t in ts]


def resample_from_map(x, sample_map, interp, interp_weights=None):
    x, sample_map, iw = _c(x, sample_map, interp_weights)
    if iw is not None:
        return mod("_weighted_resample").weighted_resample_from_map(x, sample_map, iw, interp_enum(interp))
    return mod("_resample").resample_from_map(x, sample_map, interp_enum(interp))


def resample_to_map(x, sample_map, oh, ow, interp, interp_weights=None):
    x, sample_map, iw = _c(x, sample_map, interp_weights)
    if iw is not None:
        return mod("_weighted_resample").weighted_resample_to_map(x, sample_map, iw, int(oh), int(ow),
                                                                  interp_enum(interp))
    return mod("_resample").resample_to_map(x, sample_map, int(oh), int(ow), interp_enum(interp))


def mapped_max_pool(x, sample_map, kernel_size, interp, interp_weights=None):
    x, sample_map, iw = _c(x, sample_map, interp_weights)
    if iw is not None:
        return tuple(mod("_weighted_mapped_max_pooling").weighted_mapped_max_pool(
            x, sample_map, iw, int(kernel_size), interp_enum(interp)))
    return tuple(mod("_mapped_max_pooling").mapped_max_pool(x, sample_map, int(kernel_size), interp_enum(interp)))


def mapped_max_unpool(g, idx, sample_map, ih, iw_, kernel_size, interp, interp_weights=None):
    g, idx, sample_map, iw = _c(g, idx, sample_map, interp_weights)
    if iw is not None:
        return mod("_weighted_mapped_max_pooling").weighted_mapped_max_unpool(
            g, idx, sample_map, iw, int(ih), int(iw_), int(kernel_size), interp_enum(interp))
    return mod("_mapped_max_pooling").mapped_max_unpool(g, idx, sample_map, int(ih), int(iw_), int(kernel_size),
                                                        interp_enum(interp))


def mapped_conv_forward(x, sample_map, weight, bias, kernel_size, interp, interp_weights=None):
    x, sample_map, weight, bias, iw = _c(x, sample_map, weight, bias, interp_weights)
    if iw is not None:
        return mod("_weighted_mapped_convolution").weighted_mapped_conv_forward(
            x, sample_map, iw, weight, bias, int(kernel_size), interp_enum(interp))
    return mod("_mapped_convolution").mapped_conv_forward(x, sample_map, weight, bias, int(kernel_size),
                                                          interp_enum(interp))


def mapped_conv_backward(go, sample_map, x, weight, bias, kernel_size, interp, interp_weights=None):
    go, sample_map, x, weight, bias, iw = _c(go, sample_map, x, weight, bias, interp_weights)
    if iw is not None:
        return tuple(mod("_weighted_mapped_convolution").weighted_mapped_conv_backward(
            go, sample_map, iw, x, weight, bias, int(kernel_size), interp_enum(interp)))
    return tuple(mod("_mapped_convolution").mapped_conv_backward(go, sample_map, x, weight, bias,
                                                                 int(kernel_size), interp_enum(interp)))


def mapped_transposed_conv_forward(x, sample_map, weight, bias, oh, ow, kernel_size, interp,
                                   interp_weights=None):
    x, sample_map, weight, bias, iw = _c(x, sample_map, weight, bias, interp_weights)
    if iw is not None:
        return mod("_weighted_mapped_transposed_convolution").weighted_mapped_transposed_conv_forward(
            x, sample_map, iw, weight, bias, int(oh), int(ow), int(kernel_size), interp_enum(interp))
    return mod("_mapped_transposed_convolution").mapped_transposed_conv_forward(
        x, sample_map, weight, bias, int(oh), int(ow), int(kernel_size), interp_enum(interp))


def mapped_transposed_conv_backward(go, sample_map, x, weight, bias, kernel_size, interp,
                                    interp_weights=None):
    go, sample_map, x, weight, bias, iw = _c(go, sample_map, x, weight, bias, interp_weights)
    if iw is not None:
        return tuple(mod("_weighted_mapped_transposed_convolution").weighted_mapped_transposed_conv_backward(
            go, sample_map, iw, x, weight, bias, int(kernel_size), interp_enum(interp)))
    return tuple(mod("_mapped_transposed_convolution").mapped_transposed_conv_backward(
        go, sample_map, x, weight, bias, int(kernel_size), interp_enum(interp)))


def mapped_avg_pool(x, sample_map, kernel_size, interp, interp_weights=None):
    x, sample_map, iw = _c(x, sample_map, interp_weights)
    if iw is not None:
        return mod("_weighted_mapped_avg_pooling").weighted_mapped_avg_pool(x, sample_map, iw, int(kernel_size),
                                                                            interp_enum(interp))
    return mod("_mapped_avg_pooling").mapped_avg_pool(x, sample_map, int(kernel_size), interp_enum(interp))


def mapped_avg_unpool(g, sample_map, ih, iw_, kernel_size, interp, interp_weights=None):
    g, sample_map, iw = _c(g, sample_map, interp_weights)
    if iw is not None:
        return mod("_weighted_mapped_avg_pooling").weighted_mapped_avg_unpool(g, sample_map, iw, int(ih), int(iw_),
                                                                              int(kernel_size), interp_enum(interp))
    return mod("_mapped_avg_pooling").mapped_avg_unpool(g, sample_map, int(ih), int(iw_), int(kernel_size),
                                                        interp_enum(interp))


def resample_from_uv_maps(tex, quad_idx, tex_uv, interp):
    tex, quad_idx, tex_uv = _c(tex, quad_idx, tex_uv)
    return mod("_uv_resample").resample_from_uv_maps(tex, quad_idx, tex_uv, interp_enum(interp))


def resample_to_uv_maps(x, quad_idx, tex_uv, num_textures, tex_h, tex_w, interp):
    x, quad_idx, tex_uv = _c(x, quad_idx, tex_uv)
    return mod("_uv_resample").resample_to_uv_maps(x, quad_idx, tex_uv, int(num_textures), int(tex_h), int(tex_w),
                                                   interp_enum(interp))


def voting_resample_to_map(x, sample_map, oh, ow, num_candidates):
    x, sample_map = _c(x, sample_map)
    return mod("_voting_resample").voting_resample_to_map(x, sample_map, int(oh), int(ow), int(num_candidates))
