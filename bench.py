#!/usr/bin/env python
"""Benchmark of the mapped-operator path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload encoder|pool|resample] [--precision bf16|fp32] [--batch B]

Default workload: the batch-sharded spherical encoder stack (four bilinear
mapped convolutions + ReLU on 3x3 gnomonic maps, channels 3->64->128->256->256,
512x1024 -> 128x256, global batch 64 split evenly over the GPUs), one step =
forward + backward (dInput, dW, dBias of every layer) + sum-allreduce of the
weight gradients.  Metric: algorithmic TFLOP/s (2*M*N*K of the three
contractions per layer) of the whole job.

One JSON line is printed by rank 0.  `value` is measured with the inputs
resident in HBM; `e2e` goes through the public nn.Module API with the input
batch copied from pinned host memory and the loss read back every step.
`--impl reference` times the reference's own CPU implementation (the compiled
reference modules when present, else the plain-C oracle port) on a bounded
sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "spherical-package_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if not any(len(r) >= 9 for r in self.rows):
            # the timed region was shorter than one sampling period: take one reading right after it
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=10).stdout
                self.rows = [[c.strip() for c in line.split(",")] for line in out.splitlines() if line.strip()]
            except (OSError, subprocess.TimeoutExpired):
                pass
        sm = sorted(float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit())
        if not sm:
            return None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower().startswith("active")})
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        return dict(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx) if mx else None, reasons=reasons, samples=len(sm))


def dist_setup(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, local, world


def barrier_sync(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms, world, dev):
    if world == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed_loop(step, steps, warmup, world, dev, sampler=None):
    for _ in range(warmup):
        step()
    barrier_sync(world)
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier_sync(world)
    clocks = sampler.stop() if sampler else None
    return max_over_ranks(e0.elapsed_time(e1), world, dev), clocks


# ---------------------------------------------------------------------------
# encoder stack (flagship)
# ---------------------------------------------------------------------------
def cpu_encoder_seconds(cfg, impl, images):
    """Reference CPU path (forward + backward of the four layers) on `images` images; returns seconds."""
    x = cfg["x"][:images]
    go = cfg["grad_output"][:images]
    K, it = cfg["K"], cfg["interp"]
    t0 = time.perf_counter()
    acts, ins, h = [], [], x
    for li in range(4):
        ins.append(h)
        h = impl.mapped_conv_forward(h, cfg["maps"][li], cfg["weights"][li], cfg["biases"][li], K, it).relu_()
        acts.append(h)
    g = go
    for li in reversed(range(4)):
        g = g * (acts[li] > 0)
        g, _, _ = impl.mapped_conv_backward(g, cfg["maps"][li], ins[li], cfg["weights"][li], cfg["biases"][li], K, it)
    return time.perf_counter() - t0


def pick_cpu_impl():
    from oracle import port, ref
    if ref.available():
        return ref, "reference"
    return port, "port"


def run_encoder(args, rank, local, world):
    from sphmap import capi, workloads as wl
    from sphmap.parallel import EncoderStack, GradReducer, shard_batch
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    prec = capi.BF16 if args.precision == "bf16" else capi.EXACT
    B = args.batch
    lo, hi = shard_batch(B, rank, world)
    cfg = wl.config4(B=B, H=args.height, W=2 * args.height)
    x_host = cfg["x"][lo:hi].contiguous().pin_memory()
    go = cfg["grad_output"][lo:hi].contiguous().to(dev)
    x_dev = x_host.to(dev)
    flops_step = 3 * wl.encoder_flops(B, args.height, 2 * args.height)

    # --- device-resident arm: straight through the C ABI, every conv launch bracketed by CUDA events ---
    phases = [(li, ph) for li in range(4) for ph in ("fwd", "dw", "dx", "bwd")]   # "bwd": dInput + dW in one combined call

    def new_timers():
        t = {k: [torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)] for k in phases}
        for li in range(4):   # events the combined backward call records at its internal phase boundaries
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            for e in ev:
                e.record()    # creates the handle the library records on later
            t[(li, "bwd.phases")] = ev
        return t

    stack = EncoderStack(cfg, dev, prec, hi - lo, GradReducer(mode=args.grad_exchange), None)
    per_step_timers = []

    def step():
        stack.step(x_dev, go)

    def step_timed():
        stack.timers = new_timers()
        per_step_timers.append(stack.timers)
        stack.step(x_dev, go)

    l0 = capi.lib.sph_launch_count()
    for _ in range(args.warmup):
        step()
    launches_per_step = (capi.lib.sph_launch_count() - l0) // max(args.warmup, 1)
    sampler = ClockSampler(local) if rank == 0 else None
    ms, clocks = timed_loop(step_timed, args.steps, 0, world, dev, sampler)
    # per-launch durations of the timed region itself (events were recorded on the launching stream)
    ran = sorted(stack.timed_keys)
    per_launch = {}
    for k in ran:
        if k[1] == "bwd.phases":   # split the combined backward call into its three parts
            thin = cfg["layers"][k[0]][0] * 9 <= 32   # thin layers: weight image | dW + dBias + column buffer | plan gather of dInput
            for name, i in ((("bwd.prepass", 0), ("bwd.main", 1), ("bwd.gather", 2)) if thin else (("bwd.prepass", 0), ("dx", 1), ("dw", 2))):
                per_launch[(k[0], name)] = sum(t[k][i].elapsed_time(t[k][i + 1]) for t in per_step_timers) / len(per_step_timers)
        elif not (k[1] == "bwd" and (k[0], "bwd.phases") in stack.timed_keys):
            per_launch[k] = sum(t[k][0].elapsed_time(t[k][1]) for t in per_step_timers) / len(per_step_timers)
    value = flops_step * args.steps / (ms * 1e-3) / 1e12

    # --- end-to-end arm: public nn.Module API, pinned host input copied in and loss read back per step ---
    import _spherical_distortion_ext as ext
    from spherical_distortion.nn import InterpolationType, MappedConvolution
    ext.set_precision(args.precision)
    maps = [t.to(dev) for t in cfg["maps"]]
    loss_host = [torch.empty((), dtype=torch.float32).pin_memory() for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)

    def make_e2e(fused):
        """One training step through the layer API.  fused: MappedConvolution(activation="relu") (this library's
        extension); otherwise MappedConvolution followed by torch.relu, the composition the reference's API offers."""
        mods = []
        for li, (ci, co, _, _, _) in enumerate(cfg["layers"]):
            m = MappedConvolution(ci, co, 9, InterpolationType.BILINEAR, activation="relu" if fused else None).to(dev)
            with torch.no_grad():
                m.weight.copy_(cfg["weights"][li])
                m.bias.copy_(cfg["biases"][li])
            mods.append(m)
        params = [p for m in mods for p in (m.weight, m.bias)]
        pending = []
        if world > 1 and args.grad_exchange == "layer":
            # gradient exchange as a training loop does it: each parameter's gradient is sum-allreduced in place as soon
            # as autograd has produced it, overlapping the rest of backward; the step waits for all of them at the end
            for p in params:
                p.register_post_accumulate_grad_hook(lambda t: pending.append(dist.all_reduce(t.grad, async_op=True)))
        sizes = [p.numel() for p in params]

        def exchange_bucket():
            # --grad-exchange step: all gradients as one bucket, one allreduce at the end of backward; the parameters'
            # .grad become views of the reduced bucket
            flat = torch.cat([p.grad.reshape(-1) for p in params])
            dist.all_reduce(flat)
            for p, chunk in zip(params, flat.split(sizes)):
                p.grad = chunk.view_as(p)
        # The input batch of step i+1 is copied host->device on a side stream while step i computes (what a
        # prefetching data loader does); every step's copy and its loss read-back lie inside the timed region.
        # The loss of step i is copied to pinned host memory at the end of step i and the host waits for it one step
        # later (a training loop that logs its loss one step behind), so the device does not drain between steps.
        staged = {"x": None, "ev": None}
        readback = {"i": 0, "ev": [torch.cuda.Event(), torch.cuda.Event()]}

        def stage_next():
            with torch.cuda.stream(copy_stream):
                staged["x"] = x_host.to(dev, non_blocking=True)
                staged["ev"] = torch.cuda.Event()
                staged["ev"].record(copy_stream)

        def e2e_step():
            if staged["x"] is None:
                stage_next()
            torch.cuda.current_stream().wait_event(staged["ev"])
            xb = staged["x"]
            xb.record_stream(torch.cuda.current_stream())
            stage_next()
            h = xb
            for m, sm in zip(mods, maps):
                h = m(h, sm) if fused else torch.relu(m(h, sm))
            with torch.no_grad():
                loss = torch.dot(h.reshape(-1), go.reshape(-1))   # sum(h * go) in one pass
            for p in params:
                p.grad = None
            torch.autograd.backward([h], [go])   # d loss / d h is go itself: backward is seeded with it, not with go * 1.0
            for w in pending:
                w.wait()
            pending.clear()
            if world > 1 and args.grad_exchange == "step":
                exchange_bucket()
            slot = readback["i"] & 1
            loss_host[slot].copy_(loss, non_blocking=True)
            readback["ev"][slot].record()
            if readback["i"] > 0:
                readback["ev"][slot ^ 1].synchronize()   # the previous step's loss has reached the host
            readback["i"] += 1

        return e2e_step

    del stack
    torch.cuda.empty_cache()
    e2e = {}
    for name, fused in (("e2e", True), ("e2e_unfused", False)):
        if args.skip_e2e:
            e2e[name] = (float("nan"), float("nan"))
            continue
        t_ms, _ = timed_loop(make_e2e(fused), args.steps, args.warmup, world, dev)
        e2e[name] = (t_ms, flops_step * args.steps / (t_ms * 1e-3) / 1e12)
        torch.cuda.empty_cache()
    e2e_ms, e2e_value = e2e["e2e"]
    status = capi.device_status()   # a bounded wait that gave up inside a tensor-core kernel invalidates the run
    if status != 0:
        raise SystemExit("device status %d: a bounded wait inside a tensor-core kernel gave up; results invalid" % status)

    if rank != 0:
        return None
    peaks = measured_peaks()
    # Dominant kernel = the kernel (not the single launch) with the largest share of the step.  Layers whose
    # gathered side has <= 32 (channel, slot) columns run the thin-contraction kernels (one operand block per tile on the
    # tensor cores in bf16 precision), the others the two general tcgen05 kernels (forward-type gather-GEMM for forward
    # and dInput, weight-gradient kernel for dW).
    exact = args.precision != "bf16"

    def kernel_of(li, ph):
        ci = cfg["layers"][li][0]
        if exact:   # the exact float32 path: thin register-tiled kernels for layer 1, large-tile SIMT kernels for the rest
            if ci * 9 <= 32:
                return "small_%s (SIMT, thin contraction)" % ph
            return "conv_dw128_kernel" if ph == "dw" else "conv_gemm128_kernel"
        if ci * 9 <= 32:
            return {"fwd": "tc_thin_fwd_kernel", "bwd.main": "tc_thin_bwd_kernel (dW, dBias, column buffer of dInput)",
                    "bwd.gather": "thin_plan_gather_kernel (dInput)", "bwd.prepass": "thin_wt_image_kernel",
                    "bwd": "tc_thin_bwd_kernel + thin_plan_gather_kernel (combined backward call)"}.get(
                        ph, "small_%s (SIMT, thin contraction)" % ph)
        return {"dw": "tc_dw_kernel", "bwd": "tc_gemm_kernel + tc_dw_kernel (combined backward call)",
                "bwd.prepass": "grad_image_kernel (layout pre-pass of the backward call)"}.get(ph, "tc_gemm_kernel")

    def launch_flops(li, ph):
        ci, co, _, (oh, ow), _ = cfg["layers"][li]
        return {"bwd": 2, "bwd.main": 2, "bwd.prepass": 0, "bwd.gather": 0}.get(ph, 1) * 2 * (hi - lo) * co * ci * 9 * oh * ow

    groups = {}
    for (li, ph), t in per_launch.items():
        gk = groups.setdefault(kernel_of(li, ph), [0.0, 0.0, 0])
        gk[0] += t
        gk[1] += launch_flops(li, ph)
        gk[2] += 1
    dom_kernel = max(groups, key=lambda k: groups[k][0])
    dom_ms, dom_flops_total, dom_n = groups[dom_kernel]
    tensor_peak = peaks["bf16_tflops_sustained"]
    peak_source = peaks["source"] + " bf16 sustained (kernel timed inside a long step)"
    if exact:   # no measured float32 figure exists: nominal FMA rate of the CUDA cores at the maximum SM clock
        tensor_peak = round(148 * 128 * 2 * 1.965e9 / 1e12, 1)
        peak_source = "nominal float32 FMA rate, 148 SMs x 128 lanes x 2 x 1.965 GHz (no measured figure)"
    achieved = dom_flops_total / (dom_ms * 1e-3) / 1e12
    out = {
        "metric": "mapped-conv fwd+bwd TFLOP/s", "value": round(value, 3), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16" if args.precision == "bf16" else "f32", "data": "synthetic",
        "config": {"workload": "spherical encoder stack: 4x bilinear mapped conv + ReLU on 3x3 "
                               "gnomonic maps, 3->64->128->256->256, %dx%d -> %dx%d, fwd+bwd+dW allreduce"
                               % (args.height, 2 * args.height, args.height // 4, args.height // 2),
                   "global_batch": B, "parallelism": "batch-sharded dp%d" % world, "grad_exchange": args.grad_exchange,
                   "precision": args.precision,
                   "l2": "activations (GBs per layer) exceed the 126 MB L2; no flush needed",
                   "mpix_per_s": round(B * sum(oh * ow for _, _, _, (oh, ow), _ in cfg["layers"]) * args.steps
                                       / (ms * 1e-3) / 1e6, 1)},
        "e2e": {"value": round(e2e_value, 3), "unit": "TFLOP/s", "h2d_bytes_per_step": x_host.numel() * 4 * world,
                "d2h_bytes_per_step": 4 * world, "ms_per_step": round(e2e_ms / args.steps, 3),
                "api": "spherical_distortion.nn.MappedConvolution(activation='relu') + autograd",
                "loss_readback": "every step, pinned host memory, waited for one step behind"},
        "e2e_unfused": {"value": round(e2e["e2e_unfused"][1], 3), "unit": "TFLOP/s", "h2d_bytes_per_step": x_host.numel() * 4 * world,
                        "d2h_bytes_per_step": 4 * world, "ms_per_step": round(e2e["e2e_unfused"][0] / args.steps, 3),
                        "api": "spherical_distortion.nn.MappedConvolution + torch.relu + autograd (the reference's API, no fused activation)"},
        "gpu_launches": int(launches_per_step * args.steps),
        "roofline": {"bound": "fp32" if exact else "tensor", "kernel": dom_kernel, "launches_per_step": dom_n,
                     "avg_launch_ms": round(dom_ms / dom_n, 3),
                     "algorithmic_gflop_per_launch": round(dom_flops_total / dom_n / 1e9, 1),
                     "share_of_conv_time": round(dom_ms / sum(per_launch.values()), 3),
                     "achieved": round(achieved, 2), "peak": tensor_peak, "unit": "TFLOP/s",
                     "frac": round(achieved / tensor_peak, 4),
                     # DRAM read+write of this kernel's layer-4 forward launch: 156.8 MB in an ncu capture at batch 4,
                     # scaled by local batch / 4 (activations in, activations out: proportional to the batch)
                     "traffic": None if exact else int(156.8e6 * (hi - lo) / 4),
                     "traffic_of": "layer-4 forward launch; constant from an ncu capture at batch 4 scaled by the batch, not measured in this run",
                     "peak_source": peak_source,
                     "per_launch_ms": {"L%d.%s" % (k[0] + 1, k[1]): round(v, 3) for k, v in per_launch.items()}},
        "clocks": clocks,
    }
    if world == 1 and not args.skip_extras:
        # the other benchmark workloads (max pooling, tangent-image resampling, weighted conv on a random map), a few
        # steps each, so that one default run reports every workload next to the headline
        del maps, go, x_dev
        torch.cuda.empty_cache()
        sub = argparse.Namespace(**vars(args))
        sub.steps, sub.warmup, sub.batch = max(3, min(args.steps, 5)), 3, 64
        extra = {}
        for name, fn in (("pool", run_pool), ("resample", run_resample), ("conv3", run_conv)):
            r = fn(sub, rank, local, world)
            extra[name] = {k: r[k] for k in ("metric", "value", "unit", "ms_per_step", "dtype", "config", "roofline", "cpu_baseline")}
            torch.cuda.empty_cache()
        out["extra"] = extra
    if world == 1 and not args.skip_cpu:
        impl, kind, cores = _cpu_setup()
        images = 4
        secs = cpu_encoder_seconds(cfg, impl, images)
        out["cpu_baseline"] = {"value": round(3 * wl.encoder_flops(images, args.height, 2 * args.height) / secs / 1e12, 5),
                               "unit": "TFLOP/s", "cores": cores, "kind": kind,
                               "sample": "%d image(s) of the same stack, fwd+bwd, %.1f s wall" % (images, secs)}
    return out


def run_reference(args, rank, world):
    """Reference arm: the reference's own CPU implementation of the same stack on the host cores."""
    if rank != 0:
        return None
    from sphmap import workloads as wl
    impl, kind = pick_cpu_impl()
    cores = os.cpu_count()
    torch.set_num_threads(cores)
    images = 4
    cfg = wl.config4(B=images, H=args.height, W=2 * args.height)
    for _ in range(min(args.warmup, 1)):
        cpu_encoder_seconds(cfg, impl, images)
    steps = min(args.steps, 3)
    t = sum(cpu_encoder_seconds(cfg, impl, images) for _ in range(steps))
    flops = 3 * wl.encoder_flops(images, args.height, 2 * args.height) * steps
    v = round(flops / t / 1e12, 5)
    sample = "%d image(s) per step (global batch of the GPU arm: %d), %d steps, %.1f s" % (images, args.batch, steps, t)
    return {"impl": "reference", "metric": "mapped-conv fwd+bwd TFLOP/s", "value": v, "unit": "TFLOP/s",
            "n_gpus": world, "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": round(t / steps * 1e3, 1),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "spherical encoder stack (4x bilinear mapped conv + ReLU, 3->64->128->256->256, %dx%d input) "
                                   "on the reference CPU path" % (args.height, 2 * args.height), "sample": sample},
            "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


# ---------------------------------------------------------------------------
# HBM-bound workloads: max pooling (config 2) and tangent-image resampling (config 1)
# ---------------------------------------------------------------------------
def _cpu_time(fn, reps=3):
    """Median wall time of `fn` on the host cores after one warm-up call."""
    fn()
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        ts.append(time.perf_counter() - t0)
    return sorted(ts)[len(ts) // 2]


def _cpu_setup():
    impl, kind = pick_cpu_impl()
    cores = os.cpu_count()
    torch.set_num_threads(cores)
    os.environ["OMP_NUM_THREADS"] = str(cores)
    return impl, kind, cores


def run_pool(args, rank, local, world):
    from sphmap import capi, workloads as wl
    from sphmap.parallel import shard_batch
    dev = torch.device("cuda", local)
    cfg = wl.config2(B=args.batch if args.batch != 64 else 8)
    B = cfg["x"].shape[0]
    lo, hi = shard_batch(B, rank, world)
    x, go, m = cfg["x"][lo:hi].to(dev), cfg["grad_output"][lo:hi].to(dev), cfg["map"].to(dev)
    out, idx = capi.mapped_max_pool(x, m, 9, 0)
    gin = torch.empty_like(x)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ef = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
    tf, tb, td = [], [], []
    plans = {}

    def step():
        flush.zero_()
        ef[0].record()
        capi.mapped_max_pool(x, m, 9, 0, None, out, idx)
        ef[1].record()
        flush.zero_()
        ef[2].record()
        capi.mapped_max_unpool(go, idx, m, x.shape[2], x.shape[3], 9, 0, None, gin)      # float atomics, as the reference
        ef[3].record()
        if id(m) not in plans:
            plans[id(m)] = capi.slot_plan_build(m, None, 9, 0, x.shape[2], x.shape[3])
        flush.zero_()
        ef[4].record()
        capi.mapped_max_unpool_planned(go, idx, plans[id(m)], x.shape[2], x.shape[3], 9, 0, gin)   # deterministic (plan walk)
        ef[5].record()
        torch.cuda.synchronize()
        tf.append(ef[0].elapsed_time(ef[1]))
        tb.append(ef[2].elapsed_time(ef[3]))
        td.append(ef[4].elapsed_time(ef[5]))

    for _ in range(args.warmup):
        step()
    tf.clear(), tb.clear(), td.clear()
    sampler = ClockSampler(local) if rank == 0 else None
    barrier_sync(world)
    if sampler:
        sampler.start()
    for _ in range(args.steps):
        step()
    clocks = sampler.stop() if sampler else None
    # the same kernels on a map with locality (3x3 gnomonic, stride 2: what a pooling layer of a spherical network
    # uses), same tensor sizes: shows the kernels' bandwidth when the taps are not uniformly random
    ml = wl.gnomonic_map(x.shape[2], x.shape[3], 2).to(dev)
    tf_r, tb_r, det_ms = list(tf), list(tb), sum(td) / len(td)
    tf.clear(), tb.clear(), td.clear()
    m_random, m = m, ml
    for _ in range(2 + max(3, args.steps // 2)):
        step()
    lf_ms, lb_ms = sum(tf[2:]) / len(tf[2:]), sum(tb[2:]) / len(tb[2:])
    tf[:], tb[:] = tf_r, tb_r
    m = m_random
    n = hi - lo
    fwd_bytes = x.numel() * 4 + out.numel() * 4 + idx.numel() * 8 + m.numel() * 4
    f_ms, b_ms = sum(tf) / len(tf), sum(tb) / len(tb)
    f_ms, b_ms = max_over_ranks(f_ms, world, dev), max_over_ranks(b_ms, world, dev)
    if rank != 0:
        return None
    peaks = measured_peaks()
    gbs = 2 * fwd_bytes * world / ((f_ms + b_ms) * 1e-3) / 1e9
    cpu = None
    if world == 1 and not args.skip_cpu:
        impl, kind, cores = _cpu_setup()
        cx, cm, cg = cfg["x"], cfg["map"], cfg["grad_output"]
        _, cidx = impl.mapped_max_pool(cx, cm, 9, 0)
        tfc = _cpu_time(lambda: impl.mapped_max_pool(cx, cm, 9, 0))
        tbc = _cpu_time(lambda: impl.mapped_max_unpool(cg, cidx.clamp_min(0), cm, cx.shape[2], cx.shape[3], 9, 0))
        cpu = {"value": round(2 * fwd_bytes / (tfc + tbc) / 1e9, 2), "unit": "GB/s", "cores": cores, "kind": kind,
               "sample": "the same tensors, forward %.3f s + backward %.3f s" % (tfc, tbc)}
    return {"metric": "mapped max pool fwd+bwd HBM GB/s", "cpu_baseline": cpu, "value": round(gbs, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(f_ms + b_ms, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "mapped max pool: B=%d C=64 256x512 -> 128x256, K=9, nearest, "
                                   "uniform-random map" % B, "l2": "256 MB flush before every launch", "local_batch": n},
            "gpu_launches": 2 * args.steps,
            "roofline": {"bound": "hbm", "kernel": "max_pool_kernel (forward)", "achieved": round(fwd_bytes / (f_ms * 1e-3) / 1e9, 1),
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(fwd_bytes / (f_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                         # DRAM read+write of the forward launch from an ncu capture at B=8, scaled by the local batch
                         "traffic": int(450.7e6 * n / 8), "traffic_of": "constant from an ncu capture, not measured in this run", "fwd_ms": round(f_ms, 4), "bwd_ms": round(b_ms, 4),
                         "bwd_achieved": round(fwd_bytes / (b_ms * 1e-3) / 1e9, 1),
                         "bwd_note": "value and bwd_ms use the atomic argmax backward (the reference's scheme); the "
                                     "deterministic plan-walk backward the layers use by default takes bwd_deterministic_ms",
                         "bwd_deterministic_ms": round(det_ms, 4),
                         "local_map": {"map": "3x3 gnomonic, stride 2", "fwd_ms": round(lf_ms, 4), "bwd_ms": round(lb_ms, 4),
                                       "fwd_gbs": round(fwd_bytes / (lf_ms * 1e-3) / 1e9, 1),
                                       "fwd_frac": round(fwd_bytes / (lf_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                                       "bwd_gbs": round(fwd_bytes / (lb_ms * 1e-3) / 1e9, 1)}},
            "clocks": clocks}


def _time_resample(capi, x, m, plan, H, W, steps, warmup, flush):
    y = capi.resample_from_map(x, m, 1)
    out = torch.empty_like(x)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    tg, ts = [], []
    for i in range(warmup + steps):
        flush.zero_()
        ev[0].record()
        capi.resample_from_map(x, m, 1)
        ev[1].record()
        flush.zero_()
        ev[2].record()
        capi.resample_to_map(y, plan, H, W)
        ev[3].record()
        torch.cuda.synchronize()
        if i >= warmup:
            tg.append(ev[0].elapsed_time(ev[1]))
            ts.append(ev[2].elapsed_time(ev[3]))
    del out
    return sum(tg) / len(tg), sum(ts) / len(ts)


def _resample_bytes(n, C, ns, H, W, map_numel):
    g = n * C * ns * 4 + map_numel * 4 + n * C * min(4 * ns, H * W) * 4
    sc = n * C * ns * 4 + map_numel * 4 + n * C * H * W * 4
    return g, sc


def run_resample(args, rank, local, world):
    """Tangent-image resampling (B=8), plus the same operators at B=256 so that the kernels run long enough for the
    bandwidth figure to mean something (the B=8 launches move 40-59 MB, about 6-9 us at the HBM peak)."""
    from sphmap import capi, workloads as wl
    from sphmap.parallel import shard_batch
    dev = torch.device("cuda", local)
    B = args.batch if args.batch != 64 else 8
    cfg = wl.config1(B=B)
    lo, hi = shard_batch(B, rank, world)
    x, m = cfg["x"][lo:hi].to(dev), cfg["map"].to(dev)
    H, W = cfg["out_hw"]
    plan = capi.plan_build(m, None, m.shape[0] * m.shape[1], 1, 1, H, W)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g_ms, s_ms = _time_resample(capi, x, m, plan, H, W, args.steps, args.warmup, flush)
    n, C, ns = hi - lo, x.shape[1], m.shape[0] * m.shape[1]
    g_bytes, s_bytes = _resample_bytes(n, C, ns, H, W, m.numel())
    # scaled variant: 256 images, seeded the same way
    gbig = torch.Generator().manual_seed(1)
    xb = torch.rand(256 // world, C, H, W, generator=gbig).to(dev)
    gb_ms, sb_ms = _time_resample(capi, xb, m, plan, H, W, max(3, args.steps // 2), 2, flush)
    gb_bytes, sb_bytes = _resample_bytes(xb.shape[0], C, ns, H, W, m.numel())
    g_ms, s_ms = max_over_ranks(g_ms, world, dev), max_over_ranks(s_ms, world, dev)
    gb_ms, sb_ms = max_over_ranks(gb_ms, world, dev), max_over_ranks(sb_ms, world, dev)
    if rank != 0:
        return None
    peaks = measured_peaks()
    cpu = None
    if world == 1 and not args.skip_cpu:
        impl, kind, cores = _cpu_setup()
        cx, cm = cfg["x"], cfg["map"]
        cy = impl.resample_from_map(cx, cm, 1)
        tg = _cpu_time(lambda: impl.resample_from_map(cx, cm, 1))
        ts = _cpu_time(lambda: impl.resample_to_map(cy, cm, H, W, 1))
        cpu = {"value": round((g_bytes + s_bytes) / (tg + ts) / 1e9, 2), "unit": "GB/s", "cores": cores, "kind": kind,
               "sample": "the same tensors (B=%d), gather %.3f s + scatter %.3f s" % (B, tg, ts)}
    return {"metric": "tangent-image resample HBM GB/s", "cpu_baseline": cpu, "value": round((g_bytes + s_bytes) * world / ((g_ms + s_ms) * 1e-3) / 1e9, 1),
            "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(g_ms + s_ms, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "tangent-image resampling: B=%d C=3 512x1024 <-> 20x64x64, bilinear" % B,
                       "l2": "256 MB flush before every launch"},
            "gpu_launches": 2 * args.steps,
            "roofline": {"bound": "hbm", "kernel": "resample_from_map_kernel", "achieved": round(g_bytes / (g_ms * 1e-3) / 1e9, 1),
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(g_bytes / (g_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                         # DRAM read+write of the gather launch from an ncu capture at B=8, scaled by the local batch
                         "traffic": int(49.0e6 * n / 8), "traffic_of": "constant from an ncu capture, not measured in this run", "gather_ms": round(g_ms, 4), "scatter_ms": round(s_ms, 4),
                         "scatter_achieved": round(s_bytes / (s_ms * 1e-3) / 1e9, 1),
                         "batch256": {"gather_ms": round(gb_ms, 4), "gather_gbs": round(gb_bytes / (gb_ms * 1e-3) / 1e9, 1),
                                      "gather_frac": round(gb_bytes / (gb_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                                      "scatter_ms": round(sb_ms, 4), "scatter_gbs": round(sb_bytes / (sb_ms * 1e-3) / 1e9, 1),
                                      "scatter_frac": round(sb_bytes / (sb_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)}}}


def run_conv(args, rank, local, world):
    """Weighted (4-point, nearest) mapped conv forward + backward on a uniform-random map, and the transposed conv,
    every operator timed alone with CUDA events (L2 flushed in between)."""
    from sphmap import capi, workloads as wl
    from sphmap.parallel import shard_batch
    dev = torch.device("cuda", local)
    prec = capi.BF16 if args.precision == "bf16" else capi.EXACT
    B = args.batch if args.batch != 64 else 16
    cfg = wl.config3(B=B)
    lo, hi = shard_batch(B, rank, world)
    d = lambda t: t[lo:hi].contiguous().to(dev)  # noqa: E731
    x, go, w, b, m, iw = d(cfg["x"]), d(cfg["grad_output"]), cfg["weight"].to(dev), cfg["bias"].to(dev), cfg["map"].to(dev), cfg["iw"].to(dev)
    t = cfg["t"]
    tx, tgo, tw, tb, tm, tiw = d(t["x"]), d(t["grad_output"]), t["weight"].to(dev), t["bias"].to(dev), t["map"].to(dev), t["iw"].to(dev)
    K, H, W = 9, x.shape[2], x.shape[3]
    plan = capi.plan_build(m, iw, H * W, K, 0, H, W)
    tplan = capi.plan_build(tm, tiw, tm.shape[0] * tm.shape[1], K, 0, t["oh"], t["ow"])
    ops = {
        "conv.fwd": lambda: capi.conv_forward(x, m, w, b, K, 0, iw, prec),
        "conv.dx": lambda: capi.conv_backward_input(go, plan, w, H, W, K, prec),
        "conv.dw": lambda: capi.conv_backward_weight(go, x, m, K, 0, iw, prec),
        "tconv.fwd": lambda: capi.tconv_forward(tx, tplan, tw, tb, t["oh"], t["ow"], K, prec),
        "tconv.dx": lambda: capi.tconv_backward_input(tgo, tm, tw, K, 0, tiw, prec),
        "tconv.dw": lambda: capi.tconv_backward_weight(tgo, tx, tm, K, 0, tiw, prec),
    }
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    times = {k: [] for k in ops}
    l0 = capi.lib.sph_launch_count()
    for i in range(args.warmup + args.steps):
        for k, fn in ops.items():
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times[k].append(e0.elapsed_time(e1))
    launches = (capi.lib.sph_launch_count() - l0) * args.steps // (args.warmup + args.steps)
    ms = {k: max_over_ranks(sum(v) / len(v), world, dev) for k, v in times.items()}
    if rank != 0:
        return None
    gflop_conv = 2 * B * 128 * 64 * 9 * H * W / 1e9
    gflop_t = 2 * B * 128 * 64 * 9 * (H // 2) * (W // 2) / 1e9
    conv_ms = ms["conv.fwd"] + ms["conv.dx"] + ms["conv.dw"]
    peaks = measured_peaks()
    cpu = None
    if world == 1 and not args.skip_cpu:
        impl, kind, cores = _cpu_setup()
        c1 = {k: (v[:1] if k in ("x", "grad_output") else v) for k, v in cfg.items() if torch.is_tensor(v)}
        t0 = time.perf_counter()
        impl.mapped_conv_forward(c1["x"], c1["map"], c1["weight"], c1["bias"], 9, 0, c1["iw"])
        impl.mapped_conv_backward(c1["grad_output"], c1["map"], c1["x"], c1["weight"], c1["bias"], 9, 0, c1["iw"])
        secs = time.perf_counter() - t0
        cpu = {"value": round(3 * gflop_conv / B / secs / 1e3, 4), "unit": "TFLOP/s", "cores": cores, "kind": kind,
               "sample": "1 image of the same batch, forward + backward, %.1f s" % secs}
    return {"metric": "mapped-conv fwd+bwd TFLOP/s", "cpu_baseline": cpu, "value": round(3 * gflop_conv / conv_ms, 2), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(conv_ms, 3), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if args.precision == "bf16" else "f32", "data": "synthetic",
            "config": {"workload": "weighted (P=4, nearest) mapped conv B=%d 64->128 256x512 K=9, uniform-random map; "
                                   "transposed conv 128->64 128x256->256x512" % B, "precision": args.precision,
                       "l2": "256 MB flush before every launch",
                       "mpix_per_s": round(B * H * W / (conv_ms * 1e-3) / 1e6, 1)},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "kernel": "conv forward", "achieved": round(gflop_conv / ms["conv.fwd"], 2),
                         "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": round(gflop_conv / ms["conv.fwd"] / peaks["bf16_tflops"], 4),
                         "traffic": None, "per_op_ms": {k: round(v, 3) for k, v in ms.items()},
                         "tconv_fwd_bwd_tflops": round(3 * gflop_t / (ms["tconv.fwd"] + ms["tconv.dx"] + ms["tconv.dw"]), 2)}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="encoder", choices=["encoder", "pool", "resample", "conv"])
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--batch", type=int, default=64, help="global batch")
    ap.add_argument("--height", type=int, default=512, help="input height of the encoder stack (width = 2x)")
    ap.add_argument("--skip-e2e", action="store_true", help="encoder: only the device-resident arm (for profiling runs)")
    ap.add_argument("--skip-cpu", action="store_true", help="do not time the CPU baseline")
    ap.add_argument("--grad-exchange", choices=("layer", "step"), default="step",
                    help="N > 1: allreduce dW/dBias as one bucket at the end of backward (default), or per layer as soon "
                         "as they are final (overlapped with the rest of backward)")
    ap.add_argument("--skip-extras", action="store_true", help="encoder: do not also time the pooling / resampling / weighted-conv workloads")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        out = run_reference(args, rank, world)
        if out is not None:
            print(json.dumps(out), flush=True)
        return 0
    rank, local, world = dist_setup(args.gpus)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    fn = {"encoder": run_encoder, "pool": run_pool, "resample": run_resample, "conv": run_conv}[args.workload]
    out = fn(args, rank, local, world)
    if out is not None:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
