"""ctypes binding of the C ABI declared in include/sphmap.h.

Each wrapper takes CUDA torch tensors, allocates the outputs (and the scratch
the ABI asks for) with torch, and passes raw device pointers, sizes and the
current stream to libsphmap.so.  Nothing here computes anything; if the
library is missing the import fails.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# SPHMAP_LIBRARY=checked loads the bounds-checked build of the same ABI (libsphmap_checked.so, build.py --checked)
_LIB_NAME = "libsphmap_checked.so" if os.environ.get("SPHMAP_LIBRARY", "") == "checked" else "libsphmap.so"
LIB_PATH = os.path.join(os.path.dirname(_HERE), "_spherical_distortion_ext", _LIB_NAME)

F32, F64 = 0, 1
NEAREST, BILINEAR, BISPHERICAL = 0, 1, 2
EXACT, BF16 = 0, 1
CONV_FORWARD, CONV_BACKWARD_INPUT, CONV_BACKWARD_WEIGHT = 0, 1, 2
CONV_BACKWARD = 6
TCONV_FORWARD, TCONV_BACKWARD_INPUT, TCONV_BACKWARD_WEIGHT = 3, 4, 5

SYMBOLS = [
    "sph_status_string", "sph_version", "sph_launch_count", "sph_resample_from_map", "sph_plan_bytes", "sph_plan_build",
    "sph_resample_to_map", "sph_resample_to_map_static", "sph_mapped_max_pool", "sph_mapped_max_unpool", "sph_conv_workspace_bytes",
    "sph_mapped_conv_forward", "sph_mapped_conv_backward_input", "sph_mapped_conv_backward_weight",
    "sph_mapped_tconv_forward", "sph_mapped_tconv_backward_input", "sph_mapped_tconv_backward_weight",
    "sph_mapped_conv_relu_forward", "sph_mapped_conv_relu_backward_input", "sph_mapped_conv_relu_backward_weight",
    "sph_device_status", "sph_debug_bounded_wait", "sph_mapped_max_unpool_planned", "sph_mapped_avg_pool",
    "sph_mapped_avg_unpool", "sph_resample_to_map_normalized", "sph_resample_from_uv_maps", "sph_plan_build_uv",
    "sph_voting_resample_to_map", "sph_build_kernel_map", "sph_build_is_checked", "sph_conv_companion_bytes",
    "sph_conv_companion_channels", "sph_conv_companion_fill", "sph_trace_phases", "sph_mapped_conv_forward_cl", "sph_mapped_conv_backward_cl",
]
ERR_UNSUPPORTED = 2

if not os.path.exists(LIB_PATH):
    raise ImportError("libsphmap.so not built (run spherical-package_b200/build.py): " + LIB_PATH)
lib = ctypes.CDLL(LIB_PATH)
lib.sph_status_string.restype = ctypes.c_char_p
lib.sph_status_string.argtypes = [ctypes.c_int]
lib.sph_plan_bytes.restype = ctypes.c_size_t
lib.sph_launch_count.restype = ctypes.c_ulonglong
lib.sph_conv_workspace_bytes.restype = ctypes.c_size_t
lib.sph_conv_companion_bytes.restype = ctypes.c_size_t

_vp, _i64, _int, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t


class SphError(RuntimeError):
    pass


class Unsupported(SphError):
    """A fused entry point declined the shape (SPH_ERR_UNSUPPORTED); raised only when the caller asked for no fallback."""


def _ok(rc, what):
    if rc != 0:
        raise SphError("%s failed: %s" % (what, lib.sph_status_string(rc).decode()))


def _ptr(t):
    return _vp(0 if t is None else t.data_ptr())


def _dt(t):
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.float64:
        return F64
    raise TypeError("float32/float64 only")


def _stream():
    return _vp(torch.cuda.current_stream().cuda_stream)


def _ints(*v):
    return [_i64(int(x)) for x in v]


def _P(iw):
    return 0 if iw is None else iw.shape[-1]


def _bytes(n, like):
    return torch.empty(max(int(n), 1), dtype=torch.uint8, device=like.device)


def device_status(reset=True):
    """Sticky status word of the current device: 1 if a bounded wait inside a tensor-core kernel ever gave up (the
    outputs of that launch are invalid), else 0.  Waits for the device's queued work."""
    v = ctypes.c_int(-1)
    _ok(lib.sph_device_status(ctypes.byref(v), _int(1 if reset else 0)), "sph_device_status")
    return v.value


def check_device_status():
    if device_status() != 0:
        raise SphError("a bounded wait inside a tensor-core kernel gave up: results of that launch are invalid")


def workspace_status(ws):
    """Status word (first 32 bits) of a bf16-path workspace returned by conv_workspace(); synchronises."""
    return int(ws[0][:4].view(torch.int32).item()) if ws[1] >= 4 else 0


def debug_bounded_wait(limit_ns=1000000):
    """Runs the library's self check of its bounded waits (a wait nothing satisfies, with a short limit) and returns
    the status the kernel wrote: 1 = the wait ran out and the kernel returned normally."""
    st = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    _ok(lib.sph_debug_bounded_wait(ctypes.c_ulonglong(int(limit_ns)), _ptr(st), _stream()), "sph_debug_bounded_wait")
    return int(st.item())


def resample_from_map(x, smap, interp, iw=None):
    B, C, H, W = x.shape
    MH, MW = smap.shape[:2]
    y = torch.empty(B, C, MH, MW, dtype=x.dtype, device=x.device)
    _ok(lib.sph_resample_from_map(_ptr(x), _ptr(smap), _ptr(iw), _ptr(y), *_ints(B, C, H, W, MH, MW, _P(iw)),
                                  _int(_dt(x)), _int(int(interp)), _stream()), "sph_resample_from_map")
    return y


def plan_build(smap, iw, n_src, K, interp, dstH, dstW):
    """Scatter plan for `smap` ((..., K, [P,] 2) flattened to n_src positions) pointing into a dstH x dstW image."""
    P = _P(iw)
    n = lib.sph_plan_bytes(*_ints(n_src, K, P), _int(int(interp)), *_ints(dstH, dstW), _int(_dt(smap)))
    if n == 0:
        raise SphError("sph_plan_bytes: map too large")
    plan = _bytes(n, smap)
    _ok(lib.sph_plan_build(_ptr(smap), _ptr(iw), *_ints(n_src, K, P), _int(int(interp)), *_ints(dstH, dstW),
                           _int(_dt(smap)), _ptr(plan), _sz(n), _stream()), "sph_plan_build")
    return plan


def resample_to_map(x, plan, oh, ow):
    B, C, MH, MW = x.shape
    out = torch.empty(B, C, int(oh), int(ow), dtype=x.dtype, device=x.device)
    _ok(lib.sph_resample_to_map(_ptr(x), _ptr(plan), _ptr(out), *_ints(B, C, MH, MW, oh, ow), _int(_dt(x)), _stream()),
        "sph_resample_to_map")
    return out


STATIC_SCRATCH_BYTES = 8 << 20


def resample_to_map_static(x, smap, oh, ow, interp, iw=None, out=None):
    """resample_to_map through the entry point that keeps its scratch inside the library (no allocation by the
    call itself: pass `out` to keep this wrapper from allocating the result either)."""
    B, C, MH, MW = x.shape
    if out is None:
        out = torch.empty(B, C, int(oh), int(ow), dtype=x.dtype, device=x.device)
    _ok(lib.sph_resample_to_map_static(_ptr(x), _ptr(smap), _ptr(iw), _ptr(out), *_ints(B, C, MH, MW, oh, ow, _P(iw)),
                                       _int(_dt(x)), _int(int(interp)), _stream()), "sph_resample_to_map_static")
    return out


def mapped_max_pool(x, smap, K, interp, iw=None, out=None, idx=None):
    B, C, IH, IW = x.shape
    OH, OW = smap.shape[:2]
    if out is None:
        out = torch.empty(B, C, OH, OW, dtype=x.dtype, device=x.device)
        idx = torch.empty(B, C, OH, OW, dtype=torch.int64, device=x.device)
    _ok(lib.sph_mapped_max_pool(_ptr(x), _ptr(smap), _ptr(iw), _ptr(out), _ptr(idx),
                                *_ints(B, C, IH, IW, OH, OW, K, _P(iw)), _int(_dt(x)), _int(int(interp)), _stream()),
        "sph_mapped_max_pool")
    return out, idx


def mapped_max_unpool(g, idx, smap, ih, iw_, K, interp, iw=None, out=None):
    B, C, OH, OW = g.shape
    if out is None:
        out = torch.empty(B, C, int(ih), int(iw_), dtype=g.dtype, device=g.device)
    _ok(lib.sph_mapped_max_unpool(_ptr(g), _ptr(idx), _ptr(smap), _ptr(iw), _ptr(out),
                                  *_ints(B, C, ih, iw_, OH, OW, K, _P(iw)), _int(_dt(g)), _int(int(interp)), _stream()),
        "sph_mapped_max_unpool")
    return out


def slot_plan_build(smap, iw, K, interp, dstH, dstW):
    """Scatter plan over the flattened map slots of a (OH, OW, K, [P,] 2) map (n_src = OH*OW*K positions, one slot
    each): what the deterministic argmax backward and the average-pool backward consume."""
    OH, OW = smap.shape[:2]
    return plan_build(smap, iw, OH * OW * K, 1, interp, dstH, dstW)


def mapped_max_unpool_planned(g, idx, plan, ih, iw_, K, P=0, out=None):
    B, C, OH, OW = g.shape
    if out is None:
        out = torch.empty(B, C, int(ih), int(iw_), dtype=g.dtype, device=g.device)
    _ok(lib.sph_mapped_max_unpool_planned(_ptr(g), _ptr(idx), _ptr(plan), _ptr(out), *_ints(B, C, ih, iw_, OH, OW, K, P),
                                          _int(_dt(g)), _stream()), "sph_mapped_max_unpool_planned")
    return out


def mapped_avg_pool(x, smap, K, interp, iw=None):
    B, C, IH, IW = x.shape
    OH, OW = smap.shape[:2]
    out = torch.empty(B, C, OH, OW, dtype=x.dtype, device=x.device)
    _ok(lib.sph_mapped_avg_pool(_ptr(x), _ptr(smap), _ptr(iw), _ptr(out), *_ints(B, C, IH, IW, OH, OW, K, _P(iw)),
                                _int(_dt(x)), _int(int(interp)), _stream()), "sph_mapped_avg_pool")
    return out


def mapped_avg_unpool(g, plan, ih, iw_, K):
    B, C, OH, OW = g.shape
    out = torch.empty(B, C, int(ih), int(iw_), dtype=g.dtype, device=g.device)
    _ok(lib.sph_mapped_avg_unpool(_ptr(g), _ptr(plan), _ptr(out), *_ints(B, C, ih, iw_, OH, OW, K), _int(_dt(g)), _stream()),
        "sph_mapped_avg_unpool")
    return out


def resample_to_map_normalized(x, plan, oh, ow, out=None):
    B, C, MH, MW = x.shape
    if out is None:
        out = torch.empty(B, C, int(oh), int(ow), dtype=x.dtype, device=x.device)
    _ok(lib.sph_resample_to_map_normalized(_ptr(x), _ptr(plan), _ptr(out), *_ints(B, C, MH, MW, oh, ow), _int(_dt(x)),
                                           _stream()), "sph_resample_to_map_normalized")
    return out


def resample_from_uv_maps(tex, quad, uv, interp):
    B, C, NT, TH, TW = tex.shape
    IH, IW = quad.shape
    out = torch.empty(B, C, IH, IW, dtype=tex.dtype, device=tex.device)
    _ok(lib.sph_resample_from_uv_maps(_ptr(tex), _ptr(quad), _ptr(uv), _ptr(out), *_ints(B, C, NT, TH, TW, IH, IW),
                                      _int(_dt(tex)), _int(int(interp)), _stream()), "sph_resample_from_uv_maps")
    return out


def uv_plan_build(quad, uv, NT, TH, TW, interp):
    IH, IW = quad.shape
    n = lib.sph_plan_bytes(*_ints(IH * IW, 1, 0), _int(int(interp)), *_ints(NT * TH, TW), _int(_dt(uv)))
    if n == 0:
        raise SphError("sph_plan_bytes: map too large")
    plan = _bytes(n, uv)
    _ok(lib.sph_plan_build_uv(_ptr(uv), _ptr(quad), *_ints(IH * IW, NT, TH, TW), _int(int(interp)), _int(_dt(uv)), _ptr(plan),
                              _sz(n), _stream()), "sph_plan_build_uv")
    return plan


def resample_to_uv_maps(x, quad, uv, NT, TH, TW, interp):
    plan = uv_plan_build(quad, uv, NT, TH, TW, interp)
    B, C = x.shape[:2]
    return resample_to_map(x, plan, NT * TH, TW).view(B, C, NT, TH, TW)


def voting_resample_to_map(labels, smap, oh, ow, num_candidates):
    """labels (B,C,IH,IW) int64, smap (IH,IW,2) int64 (x, y) -> (B,C,oh,ow) int64."""
    B, C, IH, IW = labels.shape
    mapf = smap.to(torch.float64)
    plan = plan_build(mapf, None, IH * IW, 1, NEAREST, oh, ow)
    out = torch.empty(B, C, int(oh), int(ow), dtype=torch.int64, device=labels.device)
    _ok(lib.sph_voting_resample_to_map(_ptr(labels), _ptr(plan), _int(F64), _ptr(out), *_ints(B, C, IH, IW, oh, ow, num_candidates),
                                       _stream()), "sph_voting_resample_to_map")
    return out


MAP_GRID, MAP_INVERSE_GNOMONIC, MAP_INVERSE_EQUIRECT = 0, 1, 2


def build_kernel_map(H, W, kh, kw, stride=1, dilation=1, kind=MAP_INVERSE_GNOMONIC, dtype=torch.float32, device="cuda"):
    OH, OW = (H + stride - 1) // stride, (W + stride - 1) // stride
    m = torch.empty(OH, OW, kh * kw, 2, dtype=dtype, device=device)
    _ok(lib.sph_build_kernel_map(_ptr(m), *_ints(H, W, kh, kw, stride, dilation), _int(kind), _int(_dt(m)), _stream()),
        "sph_build_kernel_map")
    return m


def conv_workspace(op, B, Cin, Cout, IH, IW, OH, OW, K, P, dtype, interp, precision, like):
    n = lib.sph_conv_workspace_bytes(_int(op), *_ints(B, Cin, Cout, IH, IW, OH, OW, K, P), _int(dtype),
                                     _int(int(interp)), _int(precision))
    return _bytes(n, like), n


def conv_forward(x, smap, weight, bias, K, interp, iw=None, precision=EXACT, out=None, ws=None):
    B, Cin, IH, IW = x.shape
    OH, OW = smap.shape[:2]
    Cout = weight.shape[0]
    if out is None:
        out = torch.empty(B, Cout, OH, OW, dtype=x.dtype, device=x.device)
    if ws is None:
        ws = conv_workspace(CONV_FORWARD, B, Cin, Cout, IH, IW, OH, OW, K, _P(iw), _dt(x), interp, precision, x)
    _ok(lib.sph_mapped_conv_forward(_ptr(x), _ptr(smap), _ptr(iw), _ptr(weight), _ptr(bias), _ptr(out),
                                    *_ints(B, Cin, Cout, IH, IW, OH, OW, K, _P(iw)), _int(_dt(x)), _int(int(interp)),
                                    _int(precision), _ptr(ws[0]), _sz(ws[1]), _stream()), "sph_mapped_conv_forward")
    return out


def conv_backward_input(go, plan, weight, IH, IW, K, precision=EXACT, out=None, ws=None):
    B, Cout, OH, OW = go.shape
    Cin = weight.shape[1]
    if out is None:
        out = torch.empty(B, Cin, int(IH), int(IW), dtype=go.dtype, device=go.device)
    if ws is None:
        ws = conv_workspace(CONV_BACKWARD_INPUT, B, Cin, Cout, IH, IW, OH, OW, K, 0, _dt(go), 0, precision, go)
    _ok(lib.sph_mapped_conv_backward_input(_ptr(go), _ptr(plan), _ptr(weight), _ptr(out),
                                           *_ints(B, Cin, Cout, IH, IW, OH, OW, K), _int(_dt(go)), _int(precision),
                                           _ptr(ws[0]), _sz(ws[1]), _stream()), "sph_mapped_conv_backward_input")
    return out


def conv_backward_weight(go, x, smap, K, interp, iw=None, precision=EXACT, ws=None, gw=None, gb=None):
    B, Cin, IH, IW = x.shape
    _, Cout, OH, OW = go.shape
    if gw is None:
        gw = torch.empty(Cout, Cin, K, dtype=x.dtype, device=x.device)
    if gb is None:
        gb = torch.empty(Cout, dtype=x.dtype, device=x.device)
    if ws is None:
        ws = conv_workspace(CONV_BACKWARD_WEIGHT, B, Cin, Cout, IH, IW, OH, OW, K, _P(iw), _dt(x), interp, precision, x)
    _ok(lib.sph_mapped_conv_backward_weight(_ptr(go), _ptr(x), _ptr(smap), _ptr(iw), _ptr(gw), _ptr(gb),
                                            *_ints(B, Cin, Cout, IH, IW, OH, OW, K, _P(iw)), _int(_dt(x)),
                                            _int(int(interp)), _int(precision), _ptr(ws[0]), _sz(ws[1]), _stream()),
        "sph_mapped_conv_backward_weight")
    return gw, gb


def conv_relu_forward(x, smap, weight, bias, K, interp, iw=None, precision=EXACT, out=None, ws=None):
    """max(0, conv(x) + bias) with the clamp fused into the kernels where the library supports it (see
    include/sphmap.h); elsewhere the unfused forward followed by an in-place clamp."""
    B, Cin, IH, IW = x.shape
    OH, OW = smap.shape[:2]
    Cout = weight.shape[0]
    if out is None:
        out = torch.empty(B, Cout, OH, OW, dtype=x.dtype, device=x.device)
    if ws is None:
        ws = conv_workspace(CONV_FORWARD, B, Cin, Cout, IH, IW, OH, OW, K, _P(iw), _dt(x), interp, precision, x)
    rc = lib.sph_mapped_conv_relu_forward(_ptr(x), _ptr(smap), _ptr(iw), _ptr(weight), _ptr(bias), _ptr(out),
                                          *_ints(B, Cin, Cout, IH, IW, OH, OW, K, _P(iw)), _int(_dt(x)),
                                          _int(int(interp)), _int(precision), _ptr(ws[0]), _sz(ws[1]), _stream())
    if rc == ERR_UNSUPPORTED:
        return conv_forward(x, smap, weight, bias, K, interp, iw, precision, out, ws).clamp_(min=0)
    _ok(rc, "sph_mapped_conv_relu_forward")
    return out


def conv_relu_backward_input(go, act_out, plan, weight, IH, IW, K, precision=EXACT, out=None, ws=None, fallback=True):
    """Gradient w.r.t. the input of conv_relu_forward: `go` is the gradient w.r.t. its output `act_out`.  Shapes
    the library does not fuse take one masking pass and the plain operator (or raise Unsupported if fallback=False)."""
    B, Cout, OH, OW = go.shape
    Cin = weight.shape[1]
    if out is None:
        out = torch.empty(B, Cin, int(IH), int(IW), dtype=go.dtype, device=go.device)
    if ws is None:
        ws = conv_workspace(CONV_BACKWARD_INPUT, B, Cin, Cout, IH, IW, OH, OW, K, 0, _dt(go), 0, precision, go)
    rc = lib.sph_mapped_conv_relu_backward_input(_ptr(go), _ptr(act_out), _ptr(plan), _ptr(weight), _ptr(out),
                                                 *_ints(B, Cin, Cout, IH, IW, OH, OW, K), _int(_dt(go)), _int(precision),
                                                 _ptr(ws[0]), _sz(ws[1]), _stream())
    if rc == ERR_UNSUPPORTED:
        if not fallback:
            raise Unsupported("sph_mapped_conv_relu_backward_input")
        return conv_backward_input(torch.ops.aten.threshold_backward(go, act_out, 0), plan, weight, IH, IW, K, precision, out, ws)
    _ok(rc, "sph_mapped_conv_relu_backward_input")
    return out


def conv_relu_backward_weight(go, act_out, x, smap, K, interp, iw=None, precision=EXACT, ws=None, fallback=True, gw=None,
                              gb=None):
    B, Cin, IH, IW = x.shape
    _, Cout, OH, OW = go.shape
    if gw is None:
        gw = torch.empty(Cout, Cin, K, dtype=x.dtype, device=x.device)
    if gb is None:
        gb = torch.empty(Cout, dtype=x.dtype, device=x.device)
    if ws is None:
        ws = conv_workspace(CONV_BACKWARD_WEIGHT, B, Cin, Cout, IH, IW, OH, OW, K, _P(iw), _dt(x), interp, precision, x)
    rc = lib.sph_mapped_conv_relu_backward_weight(_ptr(go), _ptr(act_out), _ptr(x), _ptr(smap), _ptr(iw), _ptr(gw), _ptr(gb),
                                                  *_ints(B, Cin, Cout, IH, IW, OH, OW, K, _P(iw)), _int(_dt(x)),
                                                  _int(int(interp)), _int(precision), _ptr(ws[0]), _sz(ws[1]), _stream())
    if rc == ERR_UNSUPPORTED:
        if not fallback:
            raise Unsupported("sph_mapped_conv_relu_backward_weight")
        return conv_backward_weight(torch.ops.aten.threshold_backward(go, act_out, 0), x, smap, K, interp, iw, precision, ws,
                                    gw, gb)
    _ok(rc, "sph_mapped_conv_relu_backward_weight")
    return gw, gb


def companion(B, C, H, W, device):
    """Zero-filled channels-last bf16 companion buffer of a (B, C, H, W) float32 activation (see include/sphmap.h)."""
    n = lib.sph_conv_companion_bytes(*_ints(B, C, H, W))
    if n == 0:
        raise SphError("sph_conv_companion_bytes: bad shape")
    return torch.zeros(n, dtype=torch.uint8, device=device)


def companion_of(x):
    """Channels-last bf16 companion of an existing float32 activation (B, C, H, W), converted now."""
    B, C, H, W = x.shape
    cl = torch.empty(lib.sph_conv_companion_bytes(*_ints(B, C, H, W)), dtype=torch.uint8, device=x.device)
    _ok(lib.sph_conv_companion_fill(_ptr(x), _ptr(cl), *_ints(B, C, H, W), _stream()), "sph_conv_companion_fill")
    return cl


def conv_forward_cl(x, x_cl, smap, weight, bias, K, interp, iw=None, precision=BF16, relu=False, out=None, out_cl=None, ws=None):
    """Forward with channels-last companions: x_cl (or None) is the companion of x, out_cl (or None) receives the
    companion of the output.  Raises Unsupported when out_cl cannot be written for this shape."""
    B, Cin, IH, IW = x.shape
    OH, OW = smap.shape[:2]
    Cout = weight.shape[0]
    if out is None:
        out = torch.empty(B, Cout, OH, OW, dtype=x.dtype, device=x.device)
    if ws is None:
        ws = conv_workspace(CONV_FORWARD, B, Cin, Cout, IH, IW, OH, OW, K, _P(iw), _dt(x), interp, precision, x)
    rc = lib.sph_mapped_conv_forward_cl(_ptr(x), _ptr(x_cl), _ptr(smap), _ptr(iw), _ptr(weight), _ptr(bias), _ptr(out), _ptr(out_cl),
                                        *_ints(B, Cin, Cout, IH, IW, OH, OW, K, _P(iw)), _int(_dt(x)), _int(int(interp)),
                                        _int(precision), _int(1 if relu else 0), _ptr(ws[0]), _sz(ws[1]), _stream())
    if rc == ERR_UNSUPPORTED:
        raise Unsupported("sph_mapped_conv_forward_cl")
    _ok(rc, "sph_mapped_conv_forward_cl")
    return out


def trace_phases(events):
    """The next conv_backward_cl call of this thread records these torch.cuda.Event objects (up to 4, created with
    enable_timing=True and recorded once before so that their handles exist) at its phase boundaries: entry,
    grad_output converted, input gradient done, weight gradient done."""
    arr = (ctypes.c_void_p * len(events))(*[ctypes.c_void_p(e.cuda_event) for e in events])
    _ok(lib.sph_trace_phases(arr, _int(len(events))), "sph_trace_phases")


def conv_backward_cl(go, act_out, x, x_cl, plan, smap, weight, K, interp, iw=None, precision=BF16, gx=None, ws=None,
                     gw=None, gb=None):
    """(grad_input, grad_weight, grad_bias) in one call; act_out (or None) masks grad_output (fused ReLU), x_cl (or
    None) is the companion of x.  Raises Unsupported for shapes that use the separate entry points."""
    B, Cin, IH, IW = x.shape
    _, Cout, OH, OW = go.shape
    if gx is None:
        gx = torch.empty_like(x)
    if gw is None:
        gw = torch.empty(Cout, Cin, K, dtype=x.dtype, device=x.device)
    if gb is None:
        gb = torch.empty(Cout, dtype=x.dtype, device=x.device)
    if ws is None:
        ws = conv_workspace(CONV_BACKWARD, B, Cin, Cout, IH, IW, OH, OW, K, _P(iw), _dt(x), interp, precision, x)
    rc = lib.sph_mapped_conv_backward_cl(_ptr(go), _ptr(act_out), _ptr(x), _ptr(x_cl), _ptr(plan), _ptr(smap), _ptr(iw),
                                         _ptr(weight), _ptr(gx), _ptr(gw), _ptr(gb), *_ints(B, Cin, Cout, IH, IW, OH, OW, K, _P(iw)),
                                         _int(_dt(x)), _int(int(interp)), _int(precision), _ptr(ws[0]), _sz(ws[1]), _stream())
    if rc == ERR_UNSUPPORTED:
        raise Unsupported("sph_mapped_conv_backward_cl")
    _ok(rc, "sph_mapped_conv_backward_cl")
    return gx, gw, gb


def tconv_forward(x, plan, weight, bias, oh, ow, K, precision=EXACT):
    B, Cin, IH, IW = x.shape
    Cout = weight.shape[1]
    out = torch.empty(B, Cout, int(oh), int(ow), dtype=x.dtype, device=x.device)
    ws = conv_workspace(TCONV_FORWARD, B, Cin, Cout, IH, IW, oh, ow, K, 0, _dt(x), 0, precision, x)
    _ok(lib.sph_mapped_tconv_forward(_ptr(x), _ptr(plan), _ptr(weight), _ptr(bias), _ptr(out),
                                     *_ints(B, Cin, Cout, IH, IW, oh, ow, K), _int(_dt(x)), _int(precision),
                                     _ptr(ws[0]), _sz(ws[1]), _stream()), "sph_mapped_tconv_forward")
    return out


def tconv_backward_input(go, smap, weight, K, interp, iw=None, precision=EXACT):
    B, Cout, OH, OW = go.shape
    IH, IW = smap.shape[:2]
    Cin = weight.shape[0]
    gx = torch.empty(B, Cin, IH, IW, dtype=go.dtype, device=go.device)
    ws = conv_workspace(TCONV_BACKWARD_INPUT, B, Cin, Cout, IH, IW, OH, OW, K, _P(iw), _dt(go), interp, precision, go)
    _ok(lib.sph_mapped_tconv_backward_input(_ptr(go), _ptr(smap), _ptr(iw), _ptr(weight), _ptr(gx),
                                            *_ints(B, Cin, Cout, IH, IW, OH, OW, K, _P(iw)), _int(_dt(go)),
                                            _int(int(interp)), _int(precision), _ptr(ws[0]), _sz(ws[1]), _stream()),
        "sph_mapped_tconv_backward_input")
    return gx


def tconv_backward_weight(go, x, smap, K, interp, iw=None, precision=EXACT):
    B, Cin, IH, IW = x.shape
    _, Cout, OH, OW = go.shape
    gw = torch.empty(Cin, Cout, K, dtype=x.dtype, device=x.device)
    gb = torch.empty(Cout, dtype=x.dtype, device=x.device)
    ws = conv_workspace(TCONV_BACKWARD_WEIGHT, B, Cin, Cout, IH, IW, OH, OW, K, _P(iw), _dt(x), interp, precision, x)
    _ok(lib.sph_mapped_tconv_backward_weight(_ptr(go), _ptr(x), _ptr(smap), _ptr(iw), _ptr(gw), _ptr(gb),
                                             *_ints(B, Cin, Cout, IH, IW, OH, OW, K, _P(iw)), _int(_dt(x)),
                                             _int(int(interp)), _int(precision), _ptr(ws[0]), _sz(ws[1]), _stream()),
        "sph_mapped_tconv_backward_weight")
    return gw, gb
