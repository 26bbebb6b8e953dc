"""Adapters that expose the CUDA library with the call signatures of oracle.port /
oracle.ref, (a) through the C ABI via ctypes and (b) through the plugin modules
of `_spherical_distortion_ext`, so parity tests can run one case on any of them."""
import torch


def _d(*ts):
    return [None if t is None else t.detach().cuda().contiguous() for t in ts]


class CApi:
    """Straight through the C ABI (sphmap.capi -> libsphmap.so)."""

    def __init__(self, precision=0):
        from sphmap import capi
        self.c, self.prec = capi, precision

    def resample_from_map(self, x, m, interp, iw=None):
        x, m, iw = _d(x, m, iw)
        return self.c.resample_from_map(x, m, interp, iw).cpu()

    def resample_to_map(self, x, m, oh, ow, interp, iw=None):
        x, m, iw = _d(x, m, iw)
        plan = self.c.plan_build(m, iw, m.shape[0] * m.shape[1], 1, interp, oh, ow)
        return self.c.resample_to_map(x, plan, oh, ow).cpu()

    def mapped_max_pool(self, x, m, K, interp, iw=None):
        x, m, iw = _d(x, m, iw)
        out, idx = self.c.mapped_max_pool(x, m, K, interp, iw)
        return out.cpu(), idx.cpu()

    def mapped_max_unpool(self, g, idx, m, ih, iw_, K, interp, iw=None):
        g, idx, m, iw = _d(g, idx, m, iw)
        return self.c.mapped_max_unpool(g, idx, m, ih, iw_, K, interp, iw).cpu()

    def mapped_conv_forward(self, x, m, w, b, K, interp, iw=None):
        x, m, w, b, iw = _d(x, m, w, b, iw)
        return self.c.conv_forward(x, m, w, b, K, interp, iw, self.prec).cpu()

    def mapped_conv_backward(self, go, m, x, w, b, K, interp, iw=None):
        go, m, x, w, iw = _d(go, m, x, w, iw)
        plan = self.c.plan_build(m, iw, m.shape[0] * m.shape[1], K, interp, x.shape[2], x.shape[3])
        gx = self.c.conv_backward_input(go, plan, w, x.shape[2], x.shape[3], K, self.prec)
        gw, gb = self.c.conv_backward_weight(go, x, m, K, interp, iw, self.prec)
        return gx.cpu(), gw.cpu(), gb.cpu()

    def mapped_transposed_conv_forward(self, x, m, w, b, oh, ow, K, interp, iw=None):
        x, m, w, b, iw = _d(x, m, w, b, iw)
        plan = self.c.plan_build(m, iw, m.shape[0] * m.shape[1], K, interp, oh, ow)
        return self.c.tconv_forward(x, plan, w, b, oh, ow, K, self.prec).cpu()

    def mapped_transposed_conv_backward(self, go, m, x, w, b, K, interp, iw=None):
        go, m, x, w, iw = _d(go, m, x, w, iw)
        gx = self.c.tconv_backward_input(go, m, w, K, interp, iw, self.prec)
        gw, gb = self.c.tconv_backward_weight(go, x, m, K, interp, iw, self.prec)
        return gx.cpu(), gw.cpu(), gb.cpu()


class Plugin:
    """Through the drop-in extension modules (the functions the reference's Python layer imports)."""

    def __init__(self):
        import _spherical_distortion_ext as ext
        from _spherical_distortion_ext import _C
        self.ext, self.m = ext, _C

    def _it(self, interp):
        return self.m.InterpolationType(int(interp))

    def resample_from_map(self, x, m, interp, iw=None):
        x, m, iw = _d(x, m, iw)
        if iw is None:
            return self.m.resample_from_map(x, m, self._it(interp)).cpu()
        return self.m.weighted_resample_from_map(x, m, iw, self._it(interp)).cpu()

    def resample_to_map(self, x, m, oh, ow, interp, iw=None):
        x, m, iw = _d(x, m, iw)
        if iw is None:
            return self.m.resample_to_map(x, m, oh, ow, self._it(interp)).cpu()
        return self.m.weighted_resample_to_map(x, m, iw, oh, ow, self._it(interp)).cpu()

    def mapped_max_pool(self, x, m, K, interp, iw=None):
        x, m, iw = _d(x, m, iw)
        r = self.m.mapped_max_pool(x, m, K, self._it(interp)) if iw is None else \
            self.m.weighted_mapped_max_pool(x, m, iw, K, self._it(interp))
        return r[0].cpu(), r[1].cpu()

    def mapped_max_unpool(self, g, idx, m, ih, iw_, K, interp, iw=None):
        g, idx, m, iw = _d(g, idx, m, iw)
        # integers arrive as 0-d tensors from the reference's autograd functions
        ih, iw_, K = torch.tensor(ih), torch.tensor(iw_), torch.tensor(K)
        if iw is None:
            return self.m.mapped_max_unpool(g, idx, m, ih, iw_, K, self._it(interp)).cpu()
        return self.m.weighted_mapped_max_unpool(g, idx, m, iw, ih, iw_, K, self._it(interp)).cpu()

    def mapped_conv_forward(self, x, m, w, b, K, interp, iw=None):
        x, m, w, b, iw = _d(x, m, w, b, iw)
        if iw is None:
            return self.m.mapped_conv_forward(x, m, w, b, K, self._it(interp)).cpu()
        return self.m.weighted_mapped_conv_forward(x, m, iw, w, b, K, self._it(interp)).cpu()

    def mapped_conv_backward(self, go, m, x, w, b, K, interp, iw=None):
        go, m, x, w, b, iw = _d(go, m, x, w, b, iw)
        K = torch.tensor(K)
        r = self.m.mapped_conv_backward(go, m, x, w, b, K, self._it(interp)) if iw is None else \
            self.m.weighted_mapped_conv_backward(go, m, iw, x, w, b, K, self._it(interp))
        return tuple(t.cpu() for t in r)

    def mapped_transposed_conv_forward(self, x, m, w, b, oh, ow, K, interp, iw=None):
        x, m, w, b, iw = _d(x, m, w, b, iw)
        if iw is None:
            return self.m.mapped_transposed_conv_forward(x, m, w, b, oh, ow, K, self._it(interp)).cpu()
        return self.m.weighted_mapped_transposed_conv_forward(x, m, iw, w, b, oh, ow, K, self._it(interp)).cpu()

    def mapped_transposed_conv_backward(self, go, m, x, w, b, K, interp, iw=None):
        go, m, x, w, b, iw = _d(go, m, x, w, b, iw)
        K = torch.tensor(K)
        r = self.m.mapped_transposed_conv_backward(go, m, x, w, b, K, self._it(interp)) if iw is None else \
            self.m.weighted_mapped_transposed_conv_backward(go, m, iw, x, w, b, K, self._it(interp))
        return tuple(t.cpu() for t in r)
