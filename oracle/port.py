"""ctypes front end of the plain-C oracle (oracle/sph_oracle.c).

TEST INFRASTRUCTURE ONLY: the checker for the CUDA library, never a fallback.
Functions take and return CPU torch tensors and use the argument order of the
reference's extension modules (ext_modules/include/layers/*.h), with the
optional interpolation weights as a trailing keyword.
"""
import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "libsph_oracle.so")
_lib = None


def build():
    subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            build()
        _lib = ctypes.CDLL(_LIB)
    return _lib


def _suf(t):
    if t.dtype == torch.float32:
        return "_f32"
    if t.dtype == torch.float64:
        return "_f64"
    raise TypeError("oracle supports float32/float64 only, got %s" % t.dtype)


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _i(*v):
    return [ctypes.c_int64(int(x)) for x in v]


def _call(name, like, *args):
    f = getattr(lib(), name + _suf(like))
    f.restype = None
    f(*args)


def _prep(*ts):
    return [None if t is None else t.detach().contiguous() for t in ts]


def _P(iw):
    return 0 if iw is None else iw.shape[-1]


def resample_from_map(x, sample_map, interp, interp_weights=None):
    x, sample_map, iw = _prep(x, sample_map, interp_weights)
    B, C, H, W = x.shape
    MH, MW = sample_map.shape[:2]
    y = torch.empty(B, C, MH, MW, dtype=x.dtype)
    _call("sph_o_resample_from_map", x, _p(x), _p(sample_map), _p(iw), _p(y),
          *_i(B, C, H, W, MH, MW, _P(iw)), ctypes.c_int(int(interp)))
    return y


def resample_to_map(x, sample_map, oh, ow, interp, interp_weights=None):
    x, sample_map, iw = _prep(x, sample_map, interp_weights)
    B, C, MH, MW = x.shape
    out = torch.empty(B, C, int(oh), int(ow), dtype=x.dtype)
    _call("sph_o_resample_to_map", x, _p(x), _p(sample_map), _p(iw), _p(out),
          *_i(B, C, MH, MW, oh, ow, _P(iw)), ctypes.c_int(int(interp)))
    return out


def mapped_max_pool(x, sample_map, kernel_size, interp, interp_weights=None, cuda_sentinel=False):
    x, sample_map, iw = _prep(x, sample_map, interp_weights)
    B, C, IH, IW = x.shape
    OH, OW = sample_map.shape[:2]
    out = torch.empty(B, C, OH, OW, dtype=x.dtype)
    idx = torch.empty(B, C, OH, OW, dtype=torch.int64)
    _call("sph_o_max_pool", x, _p(x), _p(sample_map), _p(iw), _p(out), _p(idx),
          *_i(B, C, IH, IW, OH, OW, kernel_size, _P(iw)), ctypes.c_int(int(interp)),
          ctypes.c_int(int(cuda_sentinel)))
    return out, idx


def mapped_max_unpool(g, idx, sample_map, ih, iw_, kernel_size, interp, interp_weights=None):
    g, idx, sample_map, iw = _prep(g, idx, sample_map, interp_weights)
    B, C, OH, OW = g.shape
    gin = torch.empty(B, C, int(ih), int(iw_), dtype=g.dtype)
    _call("sph_o_max_unpool", g, _p(g), _p(idx), _p(sample_map), _p(iw), _p(gin),
          *_i(B, C, ih, iw_, OH, OW, kernel_size, _P(iw)), ctypes.c_int(int(interp)))
    return gin


def mapped_conv_forward(x, sample_map, weight, bias, kernel_size, interp, interp_weights=None):
    x, sample_map, weight, bias, iw = _prep(x, sample_map, weight, bias, interp_weights)
    B, Cin, IH, IW = x.shape
    OH, OW = sample_map.shape[:2]
    Cout = weight.shape[0]
    out = torch.empty(B, Cout, OH, OW, dtype=x.dtype)
    _call("sph_o_conv_forward", x, _p(x), _p(sample_map), _p(iw), _p(weight), _p(bias), _p(out),
          *_i(B, Cin, Cout, IH, IW, OH, OW, kernel_size, _P(iw)), ctypes.c_int(int(interp)))
    return out


def mapped_conv_backward(go, sample_map, x, weight, bias, kernel_size, interp, interp_weights=None):
    go, sample_map, x, weight, iw = _prep(go, sample_map, x, weight, interp_weights)
    B, Cin, IH, IW = x.shape
    OH, OW = sample_map.shape[:2]
    Cout = weight.shape[0]
    gx, gw, gb = torch.empty_like(x), torch.empty_like(weight), torch.empty(Cout, dtype=x.dtype)
    _call("sph_o_conv_backward", x, _p(go), _p(x), _p(sample_map), _p(iw), _p(weight), _p(gx), _p(gw), _p(gb),
          *_i(B, Cin, Cout, IH, IW, OH, OW, kernel_size, _P(iw)), ctypes.c_int(int(interp)))
    return gx, gw, gb


def mapped_transposed_conv_forward(x, sample_map, weight, bias, oh, ow, kernel_size, interp,
                                   interp_weights=None):
    x, sample_map, weight, bias, iw = _prep(x, sample_map, weight, bias, interp_weights)
    B, Cin, IH, IW = x.shape
    Cout = weight.shape[1]
    out = torch.empty(B, Cout, int(oh), int(ow), dtype=x.dtype)
    _call("sph_o_tconv_forward", x, _p(x), _p(sample_map), _p(iw), _p(weight), _p(bias), _p(out),
          *_i(B, Cin, Cout, IH, IW, oh, ow, kernel_size, _P(iw)), ctypes.c_int(int(interp)))
    return out


def mapped_transposed_conv_backward(go, sample_map, x, weight, bias, kernel_size, interp,
                                    interp_weights=None):
    go, sample_map, x, weight, iw = _prep(go, sample_map, x, weight, interp_weights)
    B, Cin, IH, IW = x.shape
    Cout = weight.shape[1]
    OH, OW = go.shape[2:]
    gx, gw, gb = torch.empty_like(x), torch.empty_like(weight), torch.empty(Cout, dtype=x.dtype)
    _call("sph_o_tconv_backward", x, _p(go), _p(x), _p(sample_map), _p(iw), _p(weight), _p(gx), _p(gw), _p(gb),
          *_i(B, Cin, Cout, IH, IW, OH, OW, kernel_size, _P(iw)), ctypes.c_int(int(interp)))
    return gx, gw, gb


def mapped_avg_pool(x, sample_map, kernel_size, interp, interp_weights=None):
    x, sample_map, iw = _prep(x, sample_map, interp_weights)
    B, C, IH, IW = x.shape
    OH, OW = sample_map.shape[:2]
    out = torch.empty(B, C, OH, OW, dtype=x.dtype)
    _call("sph_o_avg_pool", x, _p(x), _p(sample_map), _p(iw), _p(out), *_i(B, C, IH, IW, OH, OW, kernel_size, _P(iw)),
          ctypes.c_int(int(interp)))
    return out


def mapped_avg_unpool(g, sample_map, ih, iw_, kernel_size, interp, interp_weights=None):
    g, sample_map, iw = _prep(g, sample_map, interp_weights)
    B, C, OH, OW = g.shape
    gin = torch.empty(B, C, int(ih), int(iw_), dtype=g.dtype)
    _call("sph_o_avg_unpool", g, _p(g), _p(sample_map), _p(iw), _p(gin), *_i(B, C, ih, iw_, OH, OW, kernel_size, _P(iw)),
          ctypes.c_int(int(interp)))
    return gin


def resample_from_uv_maps(tex, quad_idx, tex_uv, interp):
    """tex (B,C,NT,TH,TW), quad_idx (IH,IW) int64, tex_uv (IH,IW,2) -> (B,C,IH,IW)."""
    tex, quad_idx, tex_uv = _prep(tex, quad_idx, tex_uv)
    B, C, NT, TH, TW = tex.shape
    IH, IW = quad_idx.shape
    out = torch.empty(B, C, IH, IW, dtype=tex.dtype)
    _call("sph_o_resample_from_uv", tex, _p(tex), _p(quad_idx), _p(tex_uv), _p(out), *_i(B, C, NT, TH, TW, IH, IW),
          ctypes.c_int(int(interp)))
    return out


def resample_to_uv_maps(x, quad_idx, tex_uv, num_textures, tex_h, tex_w, interp):
    """x (B,C,IH,IW) -> (B,C,NT,TH,TW)."""
    x, quad_idx, tex_uv = _prep(x, quad_idx, tex_uv)
    B, C, IH, IW = x.shape
    tex = torch.empty(B, C, int(num_textures), int(tex_h), int(tex_w), dtype=x.dtype)
    _call("sph_o_resample_to_uv", x, _p(x), _p(quad_idx), _p(tex_uv), _p(tex), *_i(B, C, num_textures, tex_h, tex_w, IH, IW),
          ctypes.c_int(int(interp)))
    return tex


def voting_resample_to_map(x, sample_map, oh, ow, num_candidates):
    """x (B,C,IH,IW) int64 labels, sample_map (IH,IW,2) int64 (x, y) -> (B,C,oh,ow) int64."""
    x, sample_map = _prep(x, sample_map)
    B, C, IH, IW = x.shape
    out = torch.empty(B, C, int(oh), int(ow), dtype=torch.int64)
    f = lib().sph_o_voting_resample
    f.restype = None
    f(_p(x), _p(sample_map), _p(out), *_i(B, C, IH, IW, oh, ow, num_candidates))
    return out
