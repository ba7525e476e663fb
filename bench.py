#!/usr/bin/env python
"""Benchmark of the use_kernel shift-inference path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[3]): ResNet-18-shape DeepShift-PS inference, 256 images of
3x224x224 per GPU, 5-bit weights (10 % zero signs -> 4 weights per packed word), 4/12 fixed-point
activations, seeded synthetic weights and inputs.  One step = one forward pass over one batch.

ours:       `value`  images/s with inputs resident in HBM (integer pipeline, CUDA-graph replay,
                     logits all-gathered over NCCL when N > 1), CUDA-event timed, max over ranks;
            `e2e`    the same metric through the drop-in module API (LinearShift / Conv2dShift with
                     use_kernel=True) from pinned HOST input to HOST logits, copies inside the
                     timed region;
            `roofline`  the 3x3 convolutions of one step, CUDA-event timed, against the live
                     issue-rate probe of the pipe the kernel uses (FP32 FMA, one per shift-op); the
                     fraction of the INT32 shift+add probe is given beside it;
            `parity`    the images of the CPU baseline sample pushed through both timed objects,
                     logits compared bit for bit with the CPU reference's (outside the timed regions);
            `sweep`     a fixed subset of BASELINE.json configs[4] (shift-GEMM at K = N = 4096 and the
                     four 3x3 convolution shapes), each with its fraction of the binding peak;
            `cpu_baseline`, `clocks` (nvidia-smi samples during the timed region) and
            `gpu_launches` (counted by the library) beside them.
reference:  the reference's own CPU kernels (oracle/_ref, else the C port of them) on the host
            cores, a bounded sample of the same workload per step.
Prints exactly one JSON line on rank 0.

    python bench.py --case conv B C H OC K S P | --case gemm M K N   [--bits b] [--dense] [--act-bits n]
times one standalone layer (CUDA events, --steps launches after --warmup) and prints one JSON line:
the small cases the profiler captures are run this way.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

# torchrun sets OMP_NUM_THREADS=1 for every rank.  The reference arm runs on rank 0 alone and is
# meant to use every host core it may run on, so the limit is lifted before any OpenMP runtime loads.
if "--impl" in sys.argv and "reference" in sys.argv and os.environ.get("RANK", "0") == "0":
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "images/sec ResNet18 shift inference"
UNIT = "images/s"
BATCH_PER_GPU = 256
WORKLOAD = "resnet18_deepshift_ps_5bit_act4.12_b256x3x224x224 (BASELINE configs[3])"


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            p = [v.strip() for v in s.split(",")]
            if len(p) < 7:
                continue
            try:
                sm.append(float(p[0]))
                mx = float(p[1])
            except ValueError:
                continue
            for n, v in zip(names, p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "samples": len(sm),
                "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------ CPU reference
def _np_weights(ws):
    return [dict(shift=w['shift'].numpy(), sign=w['sign'].numpy(), bias=w['bias'].numpy()) for w in ws]


def cpu_reference(n_images=None, max_images=32, probe_marshalling=True):
    """ResNet-18 forward on the host cores with the reference's CPU kernels.

    Uses the reference's compiled deepshift_cpu module (oracle/_ref) when present -- its
    convolution_kernel / linear_kernel are called exactly as kernels.py:23,59-62 calls them, on
    pre-padded int32 tensors -- else the C port of the same loops.  With `probe_marshalling` every
    kernel call is followed by the same call on one output channel (OC = 1 / N = 1): that call pays
    the numpy -> std::vector conversion of the input and next to no arithmetic, and its time is what
    the marshalling-subtracted figure takes off.  Returns (images/s, info, input, logits)."""
    import numpy as np
    import torch
    from deepshift_b200 import workloads as W
    from oracle import oracle as O, reference_nets as R

    net = W.resnet18()
    ws = _np_weights(W.make_weights(net))
    kind = "reference" if O.ref_module() is not None else "port"
    saved = (O.conv2d, O.linear)
    probe = {"s": 0.0}

    def timed_probe(fn):
        if probe_marshalling:
            t = time.time()
            fn()
            probe["s"] += time.time() - t

    if kind == "reference":
        def conv2d(x, shift, sign, bias=None, stride=(1, 1), padding=(0, 0), zero_sign_as_plus=False):
            xp = O.pad_nchw(x, padding[0], padding[1]) if (padding[0] or padding[1]) else x
            out = O.ref_conv2d_prepadded(xp, shift, sign, bias, stride)
            timed_probe(lambda: O.ref_conv2d_prepadded(xp, shift[:1], sign[:1], None if bias is None else bias[:1], stride))
            return out

        def linear(x, shift, sign, bias=None):
            out = O.ref_linear(x, shift, sign, bias)
            timed_probe(lambda: O.ref_linear(x, shift[:1], sign[:1], None if bias is None else bias[:1]))
            return out
    else:
        def conv2d(x, shift, sign, bias=None, stride=(1, 1), padding=(0, 0), zero_sign_as_plus=False):
            out = saved[0](x, shift, sign, bias, stride, padding)
            timed_probe(lambda: saved[0](x, shift[:1], sign[:1], None if bias is None else bias[:1], stride, padding))
            return out

        def linear(x, shift, sign, bias=None):
            out = saved[1](x, shift, sign, bias)
            timed_probe(lambda: saved[1](x, shift[:1], sign[:1], None if bias is None else bias[:1]))
            return out
    O.conv2d, O.linear = conv2d, linear
    try:
        if kind == "reference" and os.environ.get("RANK", "0") == "0":
            # at::parallel_for's pool: every core this process may run on (torchrun's default is 1)
            want = int(os.environ.get("OMP_NUM_THREADS", "0")) or torch.get_num_threads()
            if want > torch.get_num_threads():
                torch.set_num_threads(want)
        cores = torch.get_num_threads() if kind == "reference" else O.num_threads()
        # The reference kernels parallelise over the batch only (at::parallel_for over images), so
        # the sample holds one image per usable core, at most max_images.
        n = max(1, min(max_images, cores if n_images is None else n_images))
        x = W.make_input(net, n)
        t0 = time.time()
        logits = R.forward(net, ws, x.numpy())
        dt = time.time() - t0 - probe["s"]      # the time of the calls a user makes
    finally:
        O.conv2d, O.linear = saved
    # threads that had work: the kernels hand out whole images
    info = {"kind": kind, "cores": int(min(cores, n)), "host_cpus": os.cpu_count(),
            "sample": "%d image(s) of the same ResNet-18 forward, %.1f s" % (n, dt)}
    if probe_marshalling:
        info["marshalling_s"] = probe["s"]
        info["value_marshalling_subtracted"] = n / max(dt - probe["s"], 1e-9)
    return n / dt, info, x, logits


def run_reference(args, rank):
    """The reference arm: the CPU kernels on a bounded sample per step.  A step is one forward pass
    of one image per host core (the kernels parallelise over images only), so it lasts as long as
    one image on one core, about 20 s; the number of timed steps is the requested one as far as
    --ref-seconds (default 150) allows, and the line reports the steps that were run."""
    if rank != 0:
        return
    t_start = time.time()
    vals, info, n = [], None, 0
    for w in range(max(1, min(args.warmup, 1))):
        cpu_reference(n_images=1, probe_marshalling=False)  # warm-up: one image
    while len(vals) < max(1, args.steps):
        v, info, x, _ = cpu_reference(probe_marshalling=(len(vals) == 0))
        vals.append(v)
        n = x.shape[0]
        per_step = (time.time() - t_start) / (len(vals) + 1)
        if time.time() - t_start + per_step > args.ref_seconds:
            break
    value = statistics.median(vals)
    world = args.gpus
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(vals), "steps_requested": args.steps, "warmup": 1, "ms_per_step": 1e3 * n / value,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch_per_gpu": BATCH_PER_GPU, "global_batch": world * BATCH_PER_GPU,
                   "parallelism": "dp%d" % world,
                   "sample_per_step": "%d images (one per host core used) of the batch of %d" % (n, BATCH_PER_GPU),
                   "note": "CPU kernels of the reference on the host cores; a step is a bounded sample of the "
                           "batch, ms_per_step is the time of that sample"},
        "cpu_baseline": {"value": value, "unit": UNIT, **info},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------ ours
def run_ours(args, rank, world, local):
    import torch
    import torch.distributed as dist
    from deepshift_b200 import kernels, sharding, workloads as W

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the shift kernels have no CPU fallback")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    net = W.resnet18()
    ws = W.make_weights(net)
    B = BATCH_PER_GPU
    x_host = W.make_input(net, B, rank=rank).pin_memory()
    x_dev = x_host.to(dev)
    pipe = W.IntPipeline(net, ws, B, dev, use_graph=True)
    gathered = torch.empty((world * B, net.layers[-1].cout), dtype=torch.float32, device=dev) if world > 1 else None

    def step():
        y = pipe.run()          # replays the captured forward pass on the static input buffer
        if world > 1:
            sharding.gather_logits_equal(y, gathered)
        return y

    pipe.x_in.copy_(x_dev)
    for _ in range(max(args.warmup, 3)):
        step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        tmax = torch.tensor([ms_total], dtype=torch.float64, device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ms_total = float(tmax.item())
    ms_per_step = ms_total / args.steps
    value = world * B * args.steps / (ms_total * 1e-3)

    # ---- end to end through the drop-in modules, host buffers, copies inside the timed region
    # (the ReLUs and residual additions that follow a shift layer go to its forward as fusion hints,
    # the max pool runs on the library's fp32 pooling kernel)
    model = W.ModuleNet(net, ws, dev, fuse=True).eval()
    model_plain = W.ModuleNet(net, ws, dev, fuse=False).eval()
    y_host = torch.empty((B, net.layers[-1].cout), dtype=torch.float32).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))

    # Double-buffered: the host->device copy of step i+1 runs on a copy stream while step i computes;
    # every step's logits are copied back and the host waits for them one step behind.
    copy_stream = torch.cuda.Stream(device=dev)
    x_bufs = [torch.empty_like(x_dev) for _ in range(2)]
    y_hosts = [torch.empty_like(y_host).pin_memory() for _ in range(2)]

    def e2e_run(nsteps, model=model):
        main = torch.cuda.current_stream(dev)
        copied = [torch.cuda.Event() for _ in range(nsteps)]
        consumed = [torch.cuda.Event() for _ in range(nsteps)]
        done = [torch.cuda.Event() for _ in range(nsteps)]
        start = torch.cuda.Event()
        start.record(main)
        copy_stream.wait_event(start)
        with torch.no_grad():
            for i in range(nsteps):
                with torch.cuda.stream(copy_stream):
                    if i >= 2:
                        copy_stream.wait_event(consumed[i - 2])
                    x_bufs[i % 2].copy_(x_host, non_blocking=True)
                    copied[i].record(copy_stream)
                main.wait_event(copied[i])
                y = model(x_bufs[i % 2])
                consumed[i].record(main)
                y_hosts[i % 2].copy_(y, non_blocking=True)
                done[i].record(main)
                if i >= 1:
                    done[i - 1].synchronize()   # the host holds the logits of the previous step
            done[nsteps - 1].synchronize()

    e2e_run(3)
    barrier()
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        tmax = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_ms = float(tmax.item())
    e2e_value = world * B * e2e_steps / (e2e_ms * 1e-3)
    # the same without the hints (every ReLU and residual addition a torch kernel of its own)
    e2e_run(2, model_plain)
    barrier()
    e0.record()
    e2e_run(e2e_steps, model_plain)
    e1.record()
    barrier()
    plain_ms = e0.elapsed_time(e1)
    if world > 1:
        tmax = torch.tensor([plain_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        plain_ms = float(tmax.item())
    e2e_plain = world * B * e2e_steps / (plain_ms * 1e-3)
    del model_plain
    clocks = sampler.stop()

    if kernels.last_kernel_error():
        raise SystemExit("a kernel gave up on a bounded wait during the timed regions: results are undefined")

    # ---- per-kernel times of one un-captured pass (CUDA events on the launching stream), for the
    # roofline of the dominant kernel: the 3x3 convolutions on the warp-specialised FP32-pipe kernel
    roofline = sweep = None
    if rank == 0:
        nograph = W.IntPipeline(net, ws, B, dev, use_graph=False)
        nograph.x_in.copy_(x_dev)
        shapes = W._trace_shapes(net)
        per_layer, all_calls = {}, []
        lib_calls = nograph.calls
        reps = 3
        for rep in range(reps + 1):
            evs = []
            for c in lib_calls:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                saved, nograph.calls = nograph.calls, [c]
                a.record()
                nograph._launch_all()
                b.record()
                nograph.calls = saved
                evs.append((c, a, b))
            torch.cuda.synchronize()
            if rep == 0:
                continue
            for c, a, b in evs:
                if c[0] in ("conv", "linear"):
                    per_layer.setdefault(c[2], []).append(a.elapsed_time(b))
                if rep == reps:
                    all_calls.append((c[0], c[2] if c[0] in ("conv", "linear") else None, a.elapsed_time(b)))
        dom_ops = dom_ms = dom_bytes = 0.0
        dom_n = 0
        for li, times in per_layer.items():
            L = net.layers[li]
            if L.kind != "conv" or L.k != 3:
                continue
            (h, w), (oh, ow) = shapes[li]
            ops = B * oh * ow * L.cout * L.cin * 9
            nbytes = 4 * (B * L.cin * h * w + L.cout * ((L.cin * 9 + 3) // 4) + L.cout + B * L.cout * oh * ow)
            dom_ops += ops
            dom_bytes += nbytes
            dom_ms += statistics.mean(times)
            dom_n += 1
        del nograph
        peak_alu = kernels.pipe_peak(0, 20000)      # shift + add issue rate, shift-ops/s
        peak_fma = kernels.pipe_peak(2, 20000)      # FFMA.RM issue rate, one term each
        achieved = dom_ops / (dom_ms * 1e-3)
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        hbm_peak, hbm_src = 6650.0, "of fallback"
        if os.path.exists(peaks_path):
            with open(peaks_path) as fh:
                hbm_peak, hbm_src = float(json.load(fh)["hbm_gbs"]), "of measured"
        roofline = {
            # the kernel issues one FP32 FMA (round toward -inf) per shift-op: neither HBM nor the
            # tensor cores bound it, the issue rate of the FMA pipe does
            "bound": "fp32_fma_issue", "kernel": "3x3 convolutions (%d launches/step)" % dom_n,
            "achieved": achieved / 1e12, "peak": peak_fma / 1e12, "unit": "Tshift-op/s (1 shift-op = 1 FFMA)",
            "frac": achieved / peak_fma,
            "peak_note": "measured live: register-only FFMA.RM probe (ds_pipe_peak mode 2)",
            "int32_alu_peak": peak_alu / 1e12, "int32_alu_frac": achieved / peak_alu,
            "int32_alu_note": "the INT32 shift+add probe (ds_pipe_peak mode 0) the target of the path is quoted "
                              "against; the kernel does not run on that pipe",
            "avg_launch_ms": dom_ms / dom_n,
            "hbm": {"achieved": dom_bytes / (dom_ms * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                    "frac": dom_bytes / (dom_ms * 1e-3) / 1e9 / hbm_peak, "peak_source": hbm_src,
                    "algorithmic_bytes_per_step": dom_bytes},
            "traffic": None,
            "traffic_source": "not measured by this run; ncu DRAM bytes of full-size layers are in profiles/",
            "per_call_ms": [[k, li, round(ms, 4)] for k, li, ms in all_calls],
        }
        if world == 1 and not args.no_sweep:
            sweep = run_sweep(peak_fma, hbm_peak)

    if rank != 0:
        return
    cpu_val, cpu_info, parity = None, None, None
    if world == 1 and not args.no_cpu_baseline:
        cpu_val, cpu_info, cpu_x, cpu_logits = cpu_reference()
        parity = check_parity(net, ws, pipe, model, x_dev, cpu_x, cpu_logits, cpu_info["kind"], dev)
    in_bytes = x_host.numel() * 4
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch_per_gpu": B, "global_batch": world * B, "parallelism": "dp%d" % world,
                   "l2": "inputs larger than L2 (%.0f MB per step per GPU)" % (in_bytes / 1e6),
                   "shift_ops_per_image": net.shift_ops(1), "Tshift_ops_per_s": value * net.shift_ops(1) / 1e12},
        "roofline": roofline,
        "cpu_baseline": ({"value": cpu_val, "unit": UNIT, **cpu_info} if cpu_info else None),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": y_host.numel() * 4,
                "api": "ModuleNet of LinearShift/Conv2dShift(use_kernel=True), pinned host input -> host logits; "
                       "ReLU / residual add after a shift layer passed to its forward as fusion hints, "
                       "max pool on the library's fp32 pooling kernel",
                "without_fusion_hints": e2e_plain, "steps": e2e_steps},
        "parity": parity,
        "sweep": sweep,
        "gpu_launches": args.steps * pipe.n_launches,
        "clocks": clocks,
    }
    print(json.dumps(line))


def check_parity(net, ws, pipe, model, x_dev, cpu_x, cpu_logits, cpu_kind, dev):
    """The images of the CPU sample through the two timed objects (the integer pipeline behind `value`,
    the module network behind `e2e`), outside the timed regions; logits compared bit for bit.

    The checker is the C restatement of the reference kernels under the canonical rule (a weight
    whose sign is 0 contributes nothing, as in the reference's linear kernel and its zero-weight
    packing).  The reference's compiled convolution kernel adds such a weight as +1
    (shift_cpu.cpp:351-353); `reference_binary` says whether a pipeline whose zero signs were set
    to +1 reproduces that binary's logits on the same images bit for bit."""
    import numpy as np
    import torch
    from deepshift_b200 import workloads as W
    from oracle import reference_nets as R
    n = min(int(cpu_x.shape[0]), 16)
    xs = cpu_x[:n]
    want = R.forward(net, _np_weights(ws), xs.numpy())
    xb = x_dev.clone()
    xb[:n] = xs.to(dev)
    got_value = pipe.run(xb)[:n].cpu().numpy()
    with torch.no_grad():
        got_e2e = model(xb)[:n].cpu().numpy()
    out = {"images": n, "checker": "oracle (C restatement of shift_cpu.cpp, pinned to the reference's golden vectors)",
           "value_path": bool(np.array_equal(got_value, want)), "e2e_path": bool(np.array_equal(got_e2e, want))}
    if cpu_kind == "reference":
        # only the convolution kernel has the quirk; the linear kernel skips zero signs (shift_cpu.cpp:190-201)
        quirk = [dict(w, sign=torch.where(w['sign'] == 0, torch.ones_like(w['sign']), w['sign']))
                 if L.kind == 'conv' else w for L, w in zip(net.layers, ws)]
        got = W.IntPipeline(net, quirk, n, dev, use_graph=False).run(xs.to(dev)).cpu().numpy()
        out["reference_binary"] = bool(np.array_equal(got, cpu_logits[:n]))
    return out


# ------------------------------------------------------------------------------------------------ standalone layers
def _sweep_weights(rng, shape, bits, dense):
    import numpy as np
    import torch
    lo = -(2 ** (bits - 1) - 1)
    shift = rng.integers(lo, 1, shape).astype(np.float32)
    if dense:
        sign = rng.choice([-1.0, 1.0], shape).astype(np.float32)
    else:
        sign = rng.choice([-1.0, 0.0, 1.0], shape, p=[0.45, 0.10, 0.45]).astype(np.float32)
    return torch.from_numpy(shift), torch.from_numpy(sign)


def _sweep_acts(rng, shape):
    import numpy as np
    import torch
    return torch.from_numpy(np.clip(np.floor(rng.normal(0, 1, shape) * 4096), -32768, 28672).astype(np.int32))


def _time_launches(fn, iters, warmup=3):
    """Average device time of one call of `fn`: `iters` calls captured into one CUDA graph (so that the
    host's launch path, tens of microseconds per call from Python, is not what gets timed for small
    layers), replayed once to warm up and once between CUDA events."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn()   # allocations of the stream's own workspace happen before capture
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(iters):
                fn()
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def run_gemm(M, K, N, bits=5, dense=False, act_bits=16, iters=10, warmup=3, dev="cuda"):
    """One shift-GEMM of BASELINE.json configs[4]: weights with shift uniform in [-(2^(b-1)-1), 0] and
    sign -1/0/+1 with P = 0.45/0.10/0.45 (or -1/+1 with `dense`), activations the int32 codes of
    round_to_fixed(N(0,1), 4, 12); through the reference-signature entry `kernels.linear`."""
    import numpy as np
    import torch
    from deepshift_b200 import kernels, utils
    rng = np.random.default_rng(20254)
    x = _sweep_acts(rng, (M, K)).to(dev)
    shift, sign = _sweep_weights(rng, (N, K), bits, dense)
    cw = utils.compress_bits(shift, sign, device=torch.device(dev))
    shift_d = shift.to(dev)
    ms = _time_launches(lambda: kernels.linear(x, shift_d, None, None, cw, act_bits=act_bits), iters, warmup)
    ops = M * K * N
    num = 32 // (cw.bits + 1)
    nbytes = 4 * (M * K + N * ((K + num - 1) // num) + M * N)
    return dict(case="gemm", M=M, K=K, N=N, weight_bits=bits, dense=dense, field_bits=cw.bits, act_bits=act_bits,
                ms=ms, Tshift_ops_per_s=ops / ms / 1e9, GBps=nbytes / ms / 1e6)


def run_conv(B, C, H, OC, k, stride, pad, bits=5, dense=False, act_bits=16, iters=10, warmup=3, dev="cuda", staged=False):
    """One square shift convolution, same distributions, through `kernels.conv2d` (int32 NCHW in and
    out), or with `staged` through `staged.conv2d` (staged fp32 NHWC operand in, int32 NHWC codes and
    the next layer's staged operand out: what a layer inside the staged pipeline does)."""
    import numpy as np
    import torch
    from deepshift_b200 import _ffi, kernels, utils
    rng = np.random.default_rng(20254)
    x = _sweep_acts(rng, (B, C, H, H)).to(dev)
    shift, sign = _sweep_weights(rng, (OC, C, k, k), bits, dense)
    cw = utils.compress_bits(shift, sign, device=torch.device(dev))
    shift_d = shift.to(dev)
    OH = (H + 2 * pad - k) // stride + 1
    if staged:
        from deepshift_b200 import staged as S
        xs = S.stage_nchw(x, 4, 12, pad, in_kind=_ffi.IN_I32)
        codes = torch.empty((B, OH, OH, OC), dtype=torch.int32, device=dev)
        nxt = S.StagedTensor(B, OH, OH, OC, 1, dev)
        ms = _time_launches(lambda: S.conv2d(xs, (OC, C, k, k), None, cw, stride, pad, relu=True, round_f32=True,
                                             out_codes=codes, out_staged=nxt), iters, warmup)
    else:
        ms = _time_launches(lambda: kernels.conv2d(x, shift_d, None, None, cw, (stride, stride), (pad, pad),
                                                   act_bits=act_bits), iters, warmup)
    ops = B * OC * OH * OH * C * k * k
    num = 32 // (cw.bits + 1)
    nbytes = 4 * (B * C * H * H + OC * ((C * k * k + num - 1) // num) + B * OC * OH * OH)
    return dict(case="conv", B=B, C=C, H=H, OC=OC, k=k, stride=stride, pad=pad, weight_bits=bits, dense=dense,
                field_bits=cw.bits, act_bits=act_bits, staged=staged, ms=ms, Tshift_ops_per_s=ops / ms / 1e9,
                GBps=nbytes / ms / 1e6)


def run_sweep(peak_fma, hbm_peak):
    """The fixed subset of configs[4] that goes into the bench line: shift-GEMM at K = N = 4096 with
    5-bit ternary weights for M = 1, 64, 1024, 8192, and the four 3x3 convolution shapes at batch 256.
    Each case carries its fraction of both peaks and names the one that binds it."""
    cases = [run_gemm(M, 4096, 4096, iters=(20 if M <= 64 else 5)) for M in (1, 64, 1024, 8192)]
    cases += [run_conv(256, C, H, C, 3, 1, 1, iters=5) for (C, H) in ((64, 56), (128, 28), (256, 14), (512, 7))]
    for c in cases:
        c["frac_fma_issue"] = c["Tshift_ops_per_s"] * 1e12 / peak_fma
        c["frac_hbm"] = c["GBps"] / hbm_peak
        # shift-ops per algorithmic byte at which the two roofs cross
        ridge = (peak_fma / 1e9) / hbm_peak
        c["bound"] = "hbm" if (c["Tshift_ops_per_s"] * 1e3 / c["GBps"]) < ridge else "fp32_fma_issue"
        c["frac"] = c["frac_hbm"] if c["bound"] == "hbm" else c["frac_fma_issue"]
    return cases


def run_case(args):
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the shift kernels have no CPU fallback")
    kw = dict(bits=args.bits, dense=args.dense, act_bits=args.act_bits, iters=args.steps, warmup=args.warmup)
    kind, dims = args.case[0], [int(v) for v in args.case[1:]]
    if kind == "all" and not dims:
        # the whole grid of BASELINE configs[4] in one process, one JSON line per case
        for dense in (False, True):
            for bits in (2, 3, 4, 5):
                for kn in (512, 1024, 2048, 4096):
                    for M in (1, 64, 1024, 8192):
                        print(json.dumps(run_gemm(M, kn, kn, bits=bits, dense=dense, act_bits=args.act_bits,
                                                  iters=(20 if M <= 64 else 5), warmup=args.warmup)), flush=True)
        for dense in (False, True):
            for (C, H) in ((64, 56), (128, 28), (256, 14), (512, 7)):
                print(json.dumps(run_conv(256, C, H, C, 3, 1, 1, bits=5, dense=dense, act_bits=args.act_bits, iters=5,
                                          warmup=args.warmup)), flush=True)
    elif kind == "gemm" and len(dims) == 3:
        print(json.dumps(run_gemm(*dims, **kw)))
    elif kind == "conv" and len(dims) == 7:
        print(json.dumps(run_conv(*dims, staged=args.staged, **kw)))
    else:
        raise SystemExit("--case conv B C H OC K S P | --case gemm M K N | --case all")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--ref-seconds", type=float, default=150.0,
                    help="reference arm: stop starting new steps when the run would pass this many seconds")
    ap.add_argument("--case", nargs="+",
                    help="time one standalone layer: conv B C H OC K S P | gemm M K N; `all`: every case of configs[4]")
    ap.add_argument("--bits", type=int, default=5)
    ap.add_argument("--dense", action="store_true")
    ap.add_argument("--act-bits", type=int, default=16)
    ap.add_argument("--staged", action="store_true", help="--case conv: the TMA-fed kernel on a staged operand")
    args = ap.parse_args()
    if args.case:
        run_case(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world > 1:
        from deepshift_b200 import sharding
        rank, world, local = sharding.init_from_env(backend="nccl")
    else:
        local = int(os.environ.get("LOCAL_RANK", "0"))
    try:
        run_ours(args, rank, world, local)
    except BaseException:
        if world > 1:
            # leave at once: the other ranks must not be kept waiting in a collective for this one
            import traceback
            traceback.print_exc()
            sys.stderr.flush()
            os._exit(1)
        raise
    if world > 1:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
