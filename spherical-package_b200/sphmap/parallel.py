"""Batch-sharded execution of mapped-operator stacks.

Every operator of the path is independent per image and the maps, weights and
biases are small, so the only sharded axis is the batch: each rank (one process
per GPU) takes a contiguous slice of the batch, runs forward / backward with no
exchange, and the single collective is the sum-allreduce of the weight and
bias gradients (NCCL on GPUs, gloo in the CPU tests): either per layer as soon
as that layer's gradients are final, overlapping the rest of backward, or as
one bucket at the end of backward (see GradReducer).
"""
import torch
import torch.distributed as dist


def shard_batch(B, rank, world):
    """Contiguous slice [lo, hi) of a batch of B images owned by `rank`; sizes differ by at most one."""
    base, rem = divmod(B, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class GradReducer:
    """Sum-allreduce of per-layer (dW, dBias), asynchronously.

    mode "layer": one message per layer, issued as soon as that layer's gradients are final, so that it overlaps
    the rest of backward.  mode "step": one message for all layers at the end of backward (a single gradient bucket).
    Gradients allocated with `buffers()` / `arena()` are views of one flat tensor, which is reduced in place with no
    packing or unpacking; any other pair is packed into a temporary and copied back in `finish()`."""

    def __init__(self, group=None, mode="layer"):
        assert mode in ("layer", "step")
        self.group = group
        self.mode = mode
        self.pending = []
        self.flats = {}
        self._arena = None
        self._arena_dirty = False
        self.enabled = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1

    def arena(self, shapes, dtype, device):
        """[(gw, gb), ...] for a list of (w_shape, b_shape): every pair adjacent, all pairs in one allocation (each
        pair starts on a 256-byte boundary; the padding between pairs is zero)."""
        sizes = [(int(torch.Size(w).numel()), int(torch.Size(b).numel())) for w, b in shapes]
        esz = torch.empty(0, dtype=dtype).element_size()
        unit = max(256 // esz, 1)
        starts, total = [], 0
        for nw, nb in sizes:
            starts.append(total)
            total += -(-(nw + nb) // unit) * unit
        flat_all = torch.zeros(total, dtype=dtype, device=device)
        out = []
        for (w_shape, b_shape), (nw, nb), lo in zip(shapes, sizes, starts):
            flat = flat_all[lo:lo + nw + nb]
            gw, gb = flat[:nw].view(w_shape), flat[nw:].view(b_shape)
            self.flats[(gw.data_ptr(), gb.data_ptr())] = flat
            out.append((gw, gb))
        self._arena = flat_all
        return out

    def buffers(self, w_shape, b_shape, dtype, device):
        """(gw, gb) of the given shapes, adjacent in one flat allocation that `submit` reduces directly."""
        nw = int(torch.Size(w_shape).numel())
        nb = int(torch.Size(b_shape).numel())
        flat = torch.empty(nw + nb, dtype=dtype, device=device)
        gw, gb = flat[:nw].view(w_shape), flat[nw:].view(b_shape)
        self.flats[(gw.data_ptr(), gb.data_ptr())] = flat
        return gw, gb

    def _in_arena(self, flat):
        a = self._arena
        return a is not None and a.data_ptr() <= flat.data_ptr() < a.data_ptr() + a.numel() * a.element_size()

    def submit(self, gw, gb):
        if not self.enabled:
            return
        flat = self.flats.get((gw.data_ptr(), gb.data_ptr()))
        if flat is not None and flat.numel() == gw.numel() + gb.numel():
            if self.mode == "step" and self._in_arena(flat):
                self._arena_dirty = True        # reduced with the whole arena in finish()
                return
            work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            self.pending.append((work, None, gw, gb))
            return
        flat = torch.cat([gw.reshape(-1), gb.reshape(-1)])
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        self.pending.append((work, flat, gw, gb))

    def finish(self):
        if self._arena_dirty:
            self._arena_dirty = False
            self.pending.append((dist.all_reduce(self._arena, op=dist.ReduceOp.SUM, group=self.group, async_op=True),
                                 None, None, None))
        for work, flat, gw, gb in self.pending:
            work.wait()
            if flat is not None:
                gw.copy_(flat[:gw.numel()].view_as(gw))
                gb.copy_(flat[gw.numel():].view_as(gb))
        self.pending = []


class EncoderStack:
    """The four-layer spherical encoder of the benchmark (mapped conv + ReLU per layer), driven straight
    through the C ABI: forward, backward (dInput, dW, dBias per layer) and gradient allreduce.  Buffers
    are allocated once; `step` enqueues one forward+backward pass and returns the loss tensor
    sum(out * grad_output) (device scalar).  With `fuse_relu` (default) the activation runs inside the
    convolution kernels (sph_mapped_conv_relu_*); without it as separate passes over the activations, the way the
    reference's operators compose."""

    def __init__(self, cfg, device, precision, local_batch, reducer=None, timers=None, fuse_relu=True, companions=None):
        from . import capi
        self.c = capi
        self.prec = precision
        self.K, self.interp = cfg["K"], cfg["interp"]
        self.layers = cfg["layers"]
        self.dev = device
        self.B = local_batch
        self.w = [t.to(device) for t in cfg["weights"]]
        self.b = [t.to(device) for t in cfg["biases"]]
        self.maps = [t.to(device) for t in cfg["maps"]]
        self.reducer = reducer
        self.fuse_relu = fuse_relu
        self.fused_bwd = [fuse_relu] * 4   # per layer: backward kernels mask the gradient themselves (else one masking pass)
        # Channels-last bf16 companions of the activations between the layers (tensor-core precision with the fused
        # ReLU only): layer i's epilogue writes the companion of its output, layer i+1 gathers from it in forward and
        # in its weight gradient, and each layer's backward is one combined call that converts grad_output once.
        self.companions = (precision == capi.BF16 and fuse_relu) if companions is None else bool(companions)
        self.out_cl = [None] * 4
        self.combined = [self.companions] * 4
        self.timers = timers          # optional {(layer, phase): [start_event, end_event]} to time single launches
        self.timed_keys = set()       # the (layer, phase) pairs that actually ran (phase "bwd" = combined backward)
        self.plans, self.acts, self.ws = [], [], {}
        f32 = dict(dtype=torch.float32, device=device)
        for li, (ci, co, (ih, iw), (oh, ow), s) in enumerate(self.layers):
            self.plans.append(capi.plan_build(self.maps[li], None, oh * ow, self.K, self.interp, ih, iw))
            self.acts.append(torch.empty(local_batch, co, oh, ow, **f32))
            if self.companions and li < 3 and co % 8 == 0:
                self.out_cl[li] = capi.companion(local_batch, co, oh, ow, device)
            for op in (capi.CONV_FORWARD, capi.CONV_BACKWARD_INPUT, capi.CONV_BACKWARD_WEIGHT, capi.CONV_BACKWARD):
                self.ws[(li, op)] = capi.conv_workspace(op, local_batch, ci, co, ih, iw, oh, ow, self.K, 0, capi.F32,
                                                        self.interp, precision, self.w[li])
        self.gx = [torch.empty(local_batch, ci, ih, iw, **f32) for ci, co, (ih, iw), _, _ in self.layers]
        # weight and bias gradients live in fixed buffers (one flat allocation per layer when a reducer owns them)
        if reducer is not None:
            pairs = reducer.arena([((co, ci, self.K), (co,)) for ci, co, _, _, _ in self.layers], torch.float32, device)
        else:
            pairs = [(torch.empty(co, ci, self.K, **f32), torch.empty(co, **f32)) for ci, co, _, _, _ in self.layers]
        self.gw, self.gb = [p[0] for p in pairs], [p[1] for p in pairs]

    def _timed(self, key, fn):
        if self.timers is not None and key in self.timers:
            self.timed_keys.add(key)
            s, e = self.timers[key]
            s.record()
            r = fn()
            e.record()
            return r
        return fn()

    def forward(self, x):
        c = self.c
        self.inputs = []
        h = x
        for li in range(4):
            self.inputs.append(h)
            if self.companions:
                x_cl = self.out_cl[li - 1] if li > 0 else None
                try:
                    out = self._timed((li, "fwd"), lambda: c.conv_forward_cl(
                        h, x_cl, self.maps[li], self.w[li], self.b[li], self.K, self.interp, None, self.prec, True,
                        out=self.acts[li], out_cl=self.out_cl[li], ws=self.ws[(li, c.CONV_FORWARD)]))
                except c.Unsupported:      # this layer cannot write a companion: the next one converts its input itself
                    self.out_cl[li] = None
                    out = self._timed((li, "fwd"), lambda: c.conv_forward_cl(
                        h, x_cl, self.maps[li], self.w[li], self.b[li], self.K, self.interp, None, self.prec, True,
                        out=self.acts[li], out_cl=None, ws=self.ws[(li, c.CONV_FORWARD)]))
                h = out
                continue
            fwd = c.conv_relu_forward if self.fuse_relu else c.conv_forward
            out = self._timed((li, "fwd"), lambda: fwd(h, self.maps[li], self.w[li], self.b[li], self.K, self.interp, None,
                                                       self.prec, out=self.acts[li], ws=self.ws[(li, c.CONV_FORWARD)]))
            h = out if self.fuse_relu else out.relu_()
        return h

    def backward(self, go):
        c = self.c
        g = go
        for li in reversed(range(4)):
            ci, co, (ih, iw), (oh, ow), s = self.layers[li]
            gw = None
            if self.combined[li]:     # one call: grad_output converted once for the input and the weight gradient
                try:
                    x_cl = self.out_cl[li - 1] if li > 0 else None
                    if self.timers is not None and (li, "bwd.phases") in self.timers:
                        c.trace_phases(self.timers[(li, "bwd.phases")])   # entry / converted / dInput done / dW done
                        self.timed_keys.add((li, "bwd.phases"))
                    gx, gw, gb = self._timed((li, "bwd"), lambda: c.conv_backward_cl(
                        g, self.acts[li], self.inputs[li], x_cl, self.plans[li], self.maps[li], self.w[li], self.K, self.interp,
                        None, self.prec, gx=self.gx[li], ws=self.ws[(li, c.CONV_BACKWARD)], gw=self.gw[li], gb=self.gb[li]))
                    if self.reducer is not None:
                        self.reducer.submit(gw, gb)
                    g = gx
                    continue
                except c.Unsupported:
                    self.combined[li] = False
            if self.fused_bwd[li]:   # the kernels read g * (activation > 0) wherever they read g
                try:
                    gw, gb = self._timed((li, "dw"), lambda: c.conv_relu_backward_weight(
                        g, self.acts[li], self.inputs[li], self.maps[li], self.K, self.interp, None, self.prec,
                        ws=self.ws[(li, c.CONV_BACKWARD_WEIGHT)], fallback=False, gw=self.gw[li], gb=self.gb[li]))
                except c.Unsupported:
                    self.fused_bwd[li] = False
            if not self.fused_bwd[li]:
                g = torch.ops.aten.threshold_backward(g, self.acts[li], 0)   # ReLU backward on the rectified activations
                gw, gb = self._timed((li, "dw"), lambda: c.conv_backward_weight(
                    g, self.inputs[li], self.maps[li], self.K, self.interp, None, self.prec,
                    ws=self.ws[(li, c.CONV_BACKWARD_WEIGHT)], gw=self.gw[li], gb=self.gb[li]))
            if self.reducer is not None:
                self.reducer.submit(gw, gb)
            if self.fused_bwd[li]:
                g = self._timed((li, "dx"), lambda: c.conv_relu_backward_input(
                    g, self.acts[li], self.plans[li], self.w[li], ih, iw, self.K, self.prec, out=self.gx[li],
                    ws=self.ws[(li, c.CONV_BACKWARD_INPUT)]))
            else:
                g = self._timed((li, "dx"), lambda: c.conv_backward_input(
                    g, self.plans[li], self.w[li], ih, iw, self.K, self.prec, out=self.gx[li],
                    ws=self.ws[(li, c.CONV_BACKWARD_INPUT)]))
        if self.reducer is not None:
            self.reducer.finish()
        return g

    def step(self, x, go):
        out = self.forward(x)
        loss = torch.dot(out.reshape(-1), go.reshape(-1))   # sum(out * go) in one pass, without the product tensor
        self.backward(go)
        return loss
