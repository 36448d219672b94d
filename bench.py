#!/usr/bin/env python
"""Benchmark of the WTConv2d forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload layers|model]

Headline workload (the BASELINE layer set): the four WTConvNeXt-T stage layers
WTConv2d(C,C,kernel_size=5,wt_levels=L) with (C,H=W,L) = (96,56,5), (192,28,4),
(384,14,3), (768,7,2), batch 128 per GPU, bf16, channels-last, x ~ N(0,1), seeded
random weights with wavelet_scale ~ U(0.05,0.2).  A "step" is one forward pass of
all four layers.  The metric is algorithmic bytes (input + output + parameters,
intermediates count zero) per second, in GB/s, summed over all ranks.

Prints ONE JSON line (rank 0).  Besides the contract keys it carries `secondary`: the other
BASELINE configurations measured in the same run (WTConvNeXt-T images/sec, the 512x512
segmentation layer, the 1-D layer, the fp32 layer set, the reference's own CUDA backend when its
offline build is present).

`--impl reference` times the reference's CPU implementation on the host cores: the unmodified
`wtconv/wtconv2d.py` module from `baseline/_ref/src` when that copy exists (with the table-only
pywt stand-in), else the operator-for-operator port in `oracle/`.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

STAGES = [(96, 56, 5), (192, 28, 4), (384, 14, 3), (768, 7, 2)]   # (C, H=W, wt_levels)
KSIZE = 5
BATCH = 128
NSETS = 4                     # rotating input sets: 4 x 144.5 MB read + the outputs written between reuses
WINDOWS = 25                  # timed windows of `steps` steps each; the line reports their median
METRIC = "wtconv2d_layer_set_algorithmic_GBps"
UNIT = "GB/s"
REF_SRC = os.path.join(ROOT, "baseline", "_ref", "src")


def param_bytes(C, L, elem, ndim=2):
    taps = KSIZE ** ndim
    sub = 4 if ndim == 2 else 2
    # (C*taps + C bias + C base_scale + L*(sub*C*taps + sub*C)) * sizeof(param)
    return (C * taps + C + C + L * (sub * C * taps + sub * C)) * elem


def layer_bytes(B, C, H, L, elem, W=None):
    return 2 * B * C * H * (H if W is None else W) * elem + param_bytes(C, L, elem)


def step_bytes(B, elem=2):
    return sum(layer_bytes(B, C, H, L, elem) for C, H, L in STAGES)


def layer_launches(B, C, H, L, code=1):
    """Kernel launches of one WTConv2d layer call (channels-last, bf16 by default), from the library."""
    import ctypes
    from wtconv_b200 import _lib
    lib = _lib.load()
    st = (ctypes.c_longlong * 4)(C * H * H, 1, H * C, C)
    out = ctypes.c_int(0)
    _lib.check(lib.wtconv2d_launch_count(B, C, H, H, 5, L, 1, code, st, st, ctypes.byref(out)),
               "wtconv2d_launch_count")
    return int(out.value)


def synthetic_state(C, L, seed, ndim=2):
    """Seeded synthetic parameters with the layer's state_dict names and shapes: conv weights and bias
    U(-1/sqrt(fan_in), 1/sqrt(fan_in)) as nn.Conv initialises them, base_scale 1, wavelet_scale U(0.05, 0.2)."""
    g = torch.Generator().manual_seed(seed)
    taps = KSIZE ** ndim
    bound = 1.0 / math.sqrt(taps)
    kshape = (KSIZE,) * ndim
    ones = (1,) * ndim

    def u(shape, lo, hi):
        return torch.rand(shape, generator=g) * (hi - lo) + lo

    sub = 4 if ndim == 2 else 2
    sd = {"base_conv.weight": u((C, 1) + kshape, -bound, bound), "base_conv.bias": u((C,), -bound, bound),
          "base_scale.weight": torch.ones((1, C) + ones)}
    for i in range(L):
        sd[f"wavelet_convs.{i}.weight"] = u((sub * C, 1) + kshape, -bound, bound)
        sd[f"wavelet_scale.{i}.weight"] = u((1, sub * C) + ones, 0.05, 0.2)
    return sd


def load_state(module, state):
    sd = module.state_dict()
    for k, v in state.items():
        sd[k] = v.reshape(sd[k].shape).to(sd[k].dtype)
    module.load_state_dict(sd, strict=True)
    return module


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.thread, self.index = [], None, None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "25",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------
# CPU arm: the reference's own layer (or the oracle port) on the host cores
# ---------------------------------------------------------------------------
def cpu_layer_factory():
    """Returns (kind, make) where make(C, L, state) -> callable x -> y on CPU tensors.
    kind "reference": the unmodified reference module; "port": the oracle restatement."""
    if os.path.isdir(os.path.join(REF_SRC, "wtconv")):
        try:
            for p in (os.path.join(ROOT, "oracle", "pywt_stub"), REF_SRC):
                if p not in sys.path:
                    sys.path.insert(0, p)
            from wtconv.wtconv2d import WTConv2d as RefWTConv2d     # the reference's own module

            def make(C, L, state):
                m = RefWTConv2d(C, C, kernel_size=KSIZE, wt_levels=L).eval()
                load_state(m, state)
                return m.to(memory_format=torch.channels_last)
            return "reference", make
        except Exception:       # noqa: BLE001 -- fall back to the port and say so in the line
            pass
    from oracle import wtconv_torch

    def make(C, L, state):
        return lambda x: wtconv_torch.wtconv2d_forward(x, state)
    return "port", make


def cpu_layer_set_seconds(batch, reps, threads, warm=1):
    """Seconds per pass of the four stage layers at `batch`, fp32 channels-last (the reference's
    fastest CPU form), with `threads` host threads.  Returns (kind, median over `reps` passes
    after `warm` untimed ones)."""
    kind, make = cpu_layer_factory()
    torch.set_num_threads(threads)
    layers = []
    for si, (C, H, L) in enumerate(STAGES):
        g = torch.Generator().manual_seed(300 + si)
        x = torch.randn(batch, C, H, H, generator=g).contiguous(memory_format=torch.channels_last)
        layers.append((x, make(C, L, synthetic_state(C, L, 100 + si))))
    times = []
    with torch.no_grad():
        for rep in range(reps + warm):
            t0 = time.perf_counter()
            for x, f in layers:
                f(x)
            if rep >= warm:
                times.append(time.perf_counter() - t0)
    return kind, statistics.median(times)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = os.cpu_count() or 1
    batch = 32                                 # bounded sample: a quarter of the per-GPU batch per step
    kind, t = cpu_layer_set_seconds(batch, args.steps, threads, warm=args.warmup)
    value = step_bytes(batch) / t / 1e9
    what = ("unmodified reference module wtconv/wtconv2d.py (pywt replaced by its four-number table)"
            if kind == "reference" else "CPU restatement of the reference forward (same ATen operator sequence)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "WTConvNeXt-T layer set (4 stage shapes), K=5, channels-last", "batch_per_step": batch,
                   "note": what + "; bytes counted at the workload's bf16 element size so that the ratio to the "
                                  "GPU arm is a speed ratio"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": f"layer set at batch {batch} (1/4 of the per-GPU batch), fp32 channels-last, "
                                   f"median of {args.steps} passes"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def build_layers(dev, dtype=torch.bfloat16):
    import wtconv_b200
    layers = []
    for si, (C, H, L) in enumerate(STAGES):
        m = wtconv_b200.WTConv2d(C, C, kernel_size=KSIZE, wt_levels=L, bias=True)
        layers.append(load_state(m, synthetic_state(C, L, 100 + si)).to(dev).to(dtype).eval())
    return layers


class Timer:
    """CUDA-event timing of `steps` calls between barriers, max over ranks."""

    def __init__(self, dev, dist):
        self.dev, self.dist = dev, dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def window(self, fn, steps, first=0, join=None):
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(first + i)
        if join is not None:
            join()                          # side streams rejoin the timed stream before the end event
        e1.record()
        self.barrier()
        ms = e0.elapsed_time(e1)
        if self.dist is not None:
            from wtconv_b200.sharding import max_over_ranks
            ms = max_over_ranks(ms, self.dev)
        return ms / steps

    def run(self, fn, steps, warmup, windows=1, join=None):
        """Returns the per-step times (ms) of `windows` windows of exactly `steps` steps each."""
        with torch.no_grad():
            for i in range(warmup):
                fn(i)
            if join is not None:
                join()
            return [self.window(fn, steps, warmup + w * steps, join) for w in range(windows)]


def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the WTConv kernels have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    from wtconv_b200 import _lib
    _lib.load()                                   # fails loudly when the CUDA library is not built
    timer = Timer(dev, dist)

    layers = build_layers(dev)
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    # one packed pinned buffer per direction: a step uploads all four inputs with one copy
    shapes = [(BATCH, C, H, H) for C, H, L in STAGES]
    numels = [BATCH * C * H * H for C, H, L in STAGES]
    host_in = torch.empty(sum(numels), dtype=torch.bfloat16).pin_memory()
    host_out = torch.empty(sum(numels), dtype=torch.bfloat16).pin_memory()
    host_in.copy_(torch.randn(sum(numels), generator=g).to(torch.bfloat16))

    def views(flat):
        """Channels-last (B,C,H,W) views of the packed buffer, one per stage."""
        out, off = [], 0
        for (B, C, H, W), n in zip(shapes, numels):
            out.append(flat[off:off + n].view(B, H, W, C).permute(0, 3, 1, 2))
            off += n
        return out

    dev_sets = []
    for k in range(NSETS):
        flat = torch.empty(sum(numels), dtype=torch.bfloat16, device=dev)
        flat.copy_(torch.randn(sum(numels), generator=g).to(torch.bfloat16))
        dev_sets.append(views(flat))
    torch.cuda.synchronize()

    def step(i):
        return [m(x) for m, x in zip(layers, dev_sets[i % NSETS])]

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    per_step = timer.run(step, args.steps, args.warmup, WINDOWS)
    # at least 0.4 s of timed steps unless fewer windows were asked for (profiler captures); every rank sees
    # the same max-over-ranks times, so all agree on the count
    with torch.no_grad():
        while WINDOWS >= 25 and sum(per_step) * args.steps < 400.0 and len(per_step) < 400:
            per_step.append(timer.window(step, args.steps, args.warmup + len(per_step) * args.steps))
    nwin = len(per_step)
    ms_step = statistics.median(per_step)

    # End to end through the public modules with HOST buffers: every step uploads the packed inputs
    # from pinned memory (one copy), runs the four forwards and downloads the four outputs.  The three
    # legs run on three streams (as a serving loop would): the upload of step i+1 and the download of
    # step i-1 overlap the kernels of step i; every step still moves all its bytes.
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    flats = [torch.empty(sum(numels), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    bufs = [views(f) for f in flats]
    out_views = views(host_out)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        k = i % 2
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_cmp[k])              # the kernels that last read flats[k] are done
            flats[k].copy_(host_in, non_blocking=True)
            ev_in[k].record(s_in)
        main.wait_event(ev_in[k])
        outs = [m(x) for m, x in zip(layers, bufs[k])]
        ev_cmp[k].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp[k])
            for ho, yv in zip(out_views, outs):
                ho.copy_(yv, non_blocking=True)
                yv.record_stream(s_out)

    def e2e_join():
        main.wait_stream(s_in)
        main.wait_stream(s_out)
    e2e_steps = max(4, args.steps // 2)
    ms_e2e = statistics.median(timer.run(e2e_step, e2e_steps, 2, 3, e2e_join))

    # the platform's floor for that traffic: the same two copies with no kernels, all ranks at once
    dflat = torch.empty(sum(numels), dtype=torch.bfloat16, device=dev)

    def copy_step(i):
        with torch.cuda.stream(s_in):
            flats[i % 2].copy_(host_in, non_blocking=True)
        with torch.cuda.stream(s_out):
            host_out.copy_(dflat, non_blocking=True)
    ms_copy = statistics.median(timer.run(copy_step, e2e_steps, 2, 3, e2e_join))

    # dominant launch: the stage-1 layer (C=96, 56x56, 5 levels), timed alone on rotating inputs
    x1 = [dev_sets[k][0] for k in range(NSETS)] + [torch.randn_like(dev_sets[0][0]) for _ in range(4)]
    ms_l1 = statistics.median(timer.run(lambda i: layers[0](x1[i % len(x1)]), max(args.steps, 20), 3, 9))
    clocks = sampler.stop() if rank == 0 else None

    secondary = None
    if not args.no_secondary:
        secondary = run_secondary(args, timer, dev, dist, rank, world)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return 0

    peak, peak_kind = load_peaks()
    total_bytes = step_bytes(BATCH) * world
    value = total_bytes / (ms_step * 1e-3) / 1e9
    C1, H1, L1 = STAGES[0]
    l1_bytes = layer_bytes(BATCH, C1, H1, L1, 2)
    achieved = l1_bytes / (ms_l1 * 1e-3) / 1e9
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "roofline_traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as f:
            traffic = json.load(f).get("stage1_bf16_bytes_per_launch")
    in_bytes = sum(numels) * 2
    threads = os.cpu_count() or 1
    sample_b = 32
    cpu_kind, t_cpu = cpu_layer_set_seconds(sample_b, 3, threads)
    cpu = {"value": step_bytes(sample_b) / t_cpu / 1e9, "unit": UNIT, "cores": threads, "kind": cpu_kind,
           "sample": f"reference forward on the host cores, layer set at batch {sample_b} "
                     f"(1/4 of the per-GPU batch), fp32 channels-last, median of 3 passes"}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "WTConvNeXt-T layer set: WTConv2d K=5, (C,H,L)=(96,56,5),(192,28,4),(384,14,3),"
                               "(768,7,2), batch 128 per GPU, bf16 storage (fp32 arithmetic), channels-last",
                   "io_dtype": "bf16",
                   "cache": f"{NSETS} rotating input sets: {NSETS * in_bytes / 1e6:.0f} MB read and as much written "
                            f"between two uses of a buffer (> 4 x L2)",
                   "timing": f"median of {nwin} windows of {args.steps} steps ({sum(per_step) * args.steps / 1e3:.2f} s timed), CUDA events, max over ranks",
                   "sharding": "batch, no collective on the data path"},
        "ms_per_step_min": min(per_step), "ms_per_step_max": max(per_step), "timed_windows": nwin,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_source": f"of {peak_kind}",
                     "kernel": "stage-1 layer call (wt2d_cl_pyramid_kernel, wt2d_cl_deep_kernel, wt2d_cl_level_kernel)",
                     "algorithmic_bytes_per_launch": l1_bytes, "ms_per_launch": ms_l1,
                     "fp32_issue_floor_ms": 2.25e9 / 35e12 * 1e3,
                     "note": "58.3 FMA per element on CUDA cores (depthwise: no tensor-core form): 2.25 GFMA at the "
                             "measured 35 TFMA/s is 0.064 ms, so frac cannot exceed 0.37 for bf16 I/O"},
        "cpu_baseline": cpu,
        "e2e": {"value": total_bytes / (ms_e2e * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": in_bytes,
                "copy_floor_ms": ms_copy,
                "note": "copy_floor_ms: the same pinned upload and download with no kernels, all ranks at once"},
        "gpu_launches": sum(layer_launches(BATCH, C, H, L) for C, H, L in STAGES) * args.steps * nwin,
        "clocks": clocks,
        "secondary": secondary,
    }
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


# ---------------------------------------------------------------------------
# Secondary measurements (the other BASELINE configurations), part of the default line
# ---------------------------------------------------------------------------
def run_secondary(args, timer, dev, dist, rank, world):
    import wtconv_b200
    peak, _ = load_peaks()
    out = {}
    with torch.no_grad():
        # config 3: WTConvNeXt-T images/sec, 256 images per GPU, bf16, whole forward as one CUDA graph
        try:
            from wtconv_b200.wtconvnext_harness import CapturedForward, WTConvNeXtTiny
            torch.manual_seed(0)
            model = WTConvNeXtTiny(wtconv_b200.WTConv2d).to(dev).to(torch.bfloat16).eval()
            model = model.to(memory_format=torch.channels_last)
            g = torch.Generator().manual_seed(77 + rank)
            xs = [torch.randn(256, 3, 224, 224, generator=g).to(torch.bfloat16)
                  .contiguous(memory_format=torch.channels_last).to(dev) for _ in range(2)]
            fwd = CapturedForward(model, xs[0])
            ms = statistics.median(timer.run(lambda i: fwd(xs[i % 2]), 5, 3, 3))
            out["wtconvnext_t_images_per_sec"] = {
                "value": 256 * world / (ms * 1e-3), "unit": "images/s", "n_gpus": world, "batch_per_gpu": 256,
                "ms_per_step": ms, "dtype": "bf16",
                "note": "timm-free WTConvNeXt-T harness, 18 WTConv2d layers on this library, other ops "
                        "cuDNN/cuBLAS, one CUDA graph per forward; synthetic 3x224x224 images"}
            del fwd, model, xs
        except Exception as e:      # noqa: BLE001
            out["wtconvnext_t_images_per_sec"] = {"unavailable": repr(e)[:200]}
        torch.cuda.empty_cache()
        if rank != 0:
            return None

        def layer_rate(m, xs, nbytes, reps=10):
            """Device time of one layer call: the calls over the rotating inputs are captured into one CUDA
            graph (a call of a small layer takes less device time than the host needs to enqueue it)."""
            for x in xs:
                m(x)                                  # plans the launch chain, folds the parameters
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for x in xs:
                        m(x)
            t = Timer(dev, None)
            ms = statistics.median(t.run(lambda i: graph.replay(), reps, 3, 3)) / len(xs)
            del graph
            return {"ms": ms, "GBps": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm": nbytes / (ms * 1e-3) / 1e9 / peak}

        # config 4: WTConv2d(256,256,5,wt_levels=5) on 512x512, bf16, 2 samples per GPU
        try:
            m = load_state(wtconv_b200.WTConv2d(256, 256, kernel_size=5, wt_levels=5), synthetic_state(256, 5, 400))
            m = m.to(dev).to(torch.bfloat16).eval()
            xs = [torch.randn(2, 256, 512, 512, device=dev, dtype=torch.bfloat16)
                  .contiguous(memory_format=torch.channels_last) for _ in range(2)]
            out["segmentation_layer_512"] = dict(layer_rate(m, xs, layer_bytes(2, 256, 512, 5, 2)),
                                                  shape="(2,256,512,512) per GPU, bf16, channels-last, wt_levels 5")
            del m, xs
        except Exception as e:      # noqa: BLE001
            out["segmentation_layer_512"] = {"unavailable": repr(e)[:200]}
        torch.cuda.empty_cache()
        # config 5: WTConv1d(64,64,5,wt_levels=4), fp32, (512,64,4096) and the odd length 4097
        for n in (4096, 4097):
            try:
                m = load_state(wtconv_b200.WTConv1d(64, 64, kernel_size=5, wt_levels=4), synthetic_state(64, 4, 500, ndim=1))
                m = m.to(dev).eval()
                t = torch.arange(n, device=dev, dtype=torch.float32)
                gsin = torch.Generator(device="cpu").manual_seed(500)
                amp = (torch.rand(512, 64, 4, generator=gsin) + 0.5).to(dev)
                freq = (torch.rand(512, 64, 4, generator=gsin) * 63 + 1).to(dev)
                phase = (torch.rand(512, 64, 4, generator=gsin) * 2 * math.pi).to(dev)
                xs = []
                for r in range(2):
                    x = torch.zeros(512, 64, n, device=dev)
                    for j in range(4):
                        x += amp[:, :, j:j + 1] * torch.sin(2 * math.pi * freq[:, :, j:j + 1] * t / n + phase[:, :, j:j + 1])
                    xs.append(x + 0.1 * torch.randn(512, 64, n, device=dev))
                nbytes = 2 * 512 * 64 * n * 4 + param_bytes(64, 4, 4, ndim=1)
                out[f"wtconv1d_len{n}"] = dict(layer_rate(m, xs, nbytes),
                                               shape=f"(512,64,{n}) fp32, sums of sinusoids + noise, wt_levels 4")
                del m, xs
            except Exception as e:      # noqa: BLE001
                out[f"wtconv1d_len{n}"] = {"unavailable": repr(e)[:200]}
            torch.cuda.empty_cache()
        # fp32 layer set and per-stage times in both dtypes
        try:
            per_stage = {}
            for dt, name, es in ((torch.bfloat16, "bf16", 2), (torch.float32, "f32", 4)):
                ls = build_layers(dev, dt)
                tot_ms, tot_b = 0.0, 0
                for (C, H, L), m in zip(STAGES, ls):
                    nb = max(2, min(8, int(600e6 / (BATCH * C * H * H * es))))
                    xs = [torch.randn(BATCH, C, H, H, device=dev, dtype=dt).contiguous(memory_format=torch.channels_last)
                          for _ in range(nb)]
                    r = layer_rate(m, xs, layer_bytes(BATCH, C, H, L, es))
                    per_stage[f"{name}_C{C}_H{H}_L{L}_us"] = r["ms"] * 1e3
                    tot_ms += r["ms"]; tot_b += layer_bytes(BATCH, C, H, L, es)
                    del xs
                per_stage[f"{name}_layer_set_GBps"] = tot_b / (tot_ms * 1e-3) / 1e9
                del ls
                torch.cuda.empty_cache()
            per_stage["note"] = "device time per layer call: CUDA graph replay over rotating inputs, batch 128, channels-last"
            out["per_stage"] = per_stage
        except Exception as e:      # noqa: BLE001
            out["per_stage"] = {"unavailable": repr(e)[:200]}
        # the reference's own fused CUDA backend (fast_wtconv), built offline for sm_100 under baseline/_ref
        out["fast_wtconv_cuda"] = time_fast_wtconv(dev)
    return out


class _StdoutToStderr:
    """Sends file descriptor 1 to stderr while third-party code runs: stdout carries the one JSON line."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)

    def __exit__(self, *exc):
        sys.stdout.flush()
        os.dup2(self.saved, 1)
        os.close(self.saved)


def time_fast_wtconv(dev):
    with _StdoutToStderr():
        return _time_fast_wtconv(dev)


def _time_fast_wtconv(dev):
    ext = os.path.join(ROOT, "baseline", "_ref", "torch_ext")
    if not os.path.isdir(os.path.join(REF_SRC, "fast_wtconv")) or not os.path.isdir(ext):
        return {"unavailable": "baseline/_ref holds no offline build of fast_wtconv (baseline/time_fast_wtconv.py --install)"}
    try:
        os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
        os.environ.setdefault("TORCH_EXTENSIONS_DIR", ext)
        os.environ.setdefault("HAAR_MAX_K", "5")
        if REF_SRC not in sys.path:
            sys.path.insert(0, REF_SRC)
        from fast_wtconv.wtconv_cuda import WTConv2d as FastWTConv2d
        res = {"note": "reference's fused CUDA backend, NCHW bf16, batch 128, CUDA events including host launch time"}
        for C, H, L in STAGES:
            ref = FastWTConv2d(C, C, 5, 1, L, True).to(dev).to(torch.bfloat16).eval()
            xs = [torch.randn(BATCH, C, H, H, device=dev, dtype=torch.bfloat16) for _ in range(2)]
            ms = statistics.median(Timer(dev, None).run(lambda i: ref(xs[i % 2]), 10, 3, 3))
            res[f"C{C}_H{H}_L{L}_us"] = ms * 1e3
            del ref, xs
        return res
    except Exception as e:      # noqa: BLE001
        return {"unavailable": repr(e)[:300]}


# ---------------------------------------------------------------------------
# Alternative headline: full WTConvNeXt-T inference (images/sec), `--workload model`
# ---------------------------------------------------------------------------
class _CpuLayer(torch.nn.Module):
    """CPU arm of the model workload: the layer's parameters run through the reference forward."""

    def __init__(self, c_in, c_out, kernel_size=5, stride=1, bias=True, wt_levels=1):
        super().__init__()
        import wtconv_b200
        self.inner = wtconv_b200.WTConv2d(c_in, c_out, kernel_size=kernel_size, stride=stride, bias=bias,
                                          wt_levels=wt_levels)

    def forward(self, x):
        from oracle import wtconv_torch
        return wtconv_torch.wtconv2d_forward(
            x, {k: v for k, v in self.inner.state_dict().items() if "filter" not in k})


def cpu_model_images_per_sec(batch, reps, threads):
    from wtconv_b200.wtconvnext_harness import WTConvNeXtTiny
    torch.set_num_threads(threads)
    torch.manual_seed(0)
    model = WTConvNeXtTiny(_CpuLayer).eval()
    x = torch.randn(batch, 3, 224, 224).contiguous(memory_format=torch.channels_last)
    ts = []
    with torch.no_grad():
        for rep in range(reps + 1):
            t0 = time.perf_counter()
            model(x)
            if rep:
                ts.append(time.perf_counter() - t0)
    return batch / statistics.median(ts)


def run_model(args):
    """WTConvNeXt-T (depths 3-3-9-3, dims 96-192-384-768, 18 WTConv2d layers), random init from seed 0,
    synthetic N(0,1) 3x224x224 images, bf16, batch per GPU (BASELINE config 3: 256)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    batch = args.batch if args.batch != 128 else 256
    metric = "wtconvnext_t_inference_images_per_sec"
    threads = os.cpu_count() or 1
    if args.impl == "reference":
        if rank != 0:
            return 0
        v = cpu_model_images_per_sec(8, max(1, args.steps), threads)
        print(json.dumps({"impl": "reference", "metric": metric, "value": v, "unit": "images/s", "n_gpus": args.gpus,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": 8e3 / v,
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                          "data": "synthetic", "config": {"workload": "WTConvNeXt-T inference, batch 8 sample"},
                          "cpu_baseline": {"value": v, "unit": "images/s", "cores": threads, "kind": "port",
                                           "sample": "timm-free harness with oracle layers, batch 8, fp32"},
                          "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return 0
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    import wtconv_b200
    from wtconv_b200.wtconvnext_harness import CapturedForward, WTConvNeXtTiny
    timer = Timer(dev, dist)
    torch.manual_seed(0)
    model = WTConvNeXtTiny(wtconv_b200.WTConv2d).to(dev).to(torch.bfloat16).eval()
    model = model.to(memory_format=torch.channels_last)
    g = torch.Generator().manual_seed(77 + rank)
    host = [torch.randn(batch, 3, 224, 224, generator=g).to(torch.bfloat16)
            .contiguous(memory_format=torch.channels_last).pin_memory() for _ in range(2)]
    xs = [h.to(dev) for h in host]
    host_out = torch.empty(batch, 1000, dtype=torch.bfloat16).pin_memory()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # the whole forward is one CUDA graph; a step copies the batch into its input buffer and replays
    fwd = CapturedForward(model, xs[0])
    ms = statistics.median(timer.run(lambda i: fwd(xs[i % 2]), args.steps, args.warmup, 5))
    ms_e2e = statistics.median(timer.run(lambda i: host_out.copy_(fwd(host[i % 2]), non_blocking=True),
                                         max(2, args.steps // 2), 2, 3))
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        cpu_v = cpu_model_images_per_sec(8, 2, threads)
        print(json.dumps({
            "metric": metric, "value": batch * world / (ms * 1e-3), "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "WTConvNeXt-T inference (timm-free harness, 18 WTConv2d layers on the sm_100a "
                                   "kernels, other ops cuDNN/cuBLAS; forward replayed as one CUDA graph)", "batch_per_gpu": batch,
                       "note": "published 536.71 img/s (logs/val_tiny.out:31) is fp32 with data loading on "
                               "unstated hardware: not comparable, vs_baseline stays null"},
            "cpu_baseline": {"value": cpu_v, "unit": "images/s", "cores": threads, "kind": "port",
                             "sample": "same harness with oracle layers on the host cores, batch 8, fp32"},
            "e2e": {"value": batch * world / (ms_e2e * 1e-3), "unit": "images/s",
                    "h2d_bytes_per_step": host[0].numel() * 2, "d2h_bytes_per_step": host_out.numel() * 2},
            "gpu_launches": sum(d * layer_launches(batch, C, H, L)
                                for d, (C, H, L) in zip((3, 3, 9, 3), STAGES)) * args.steps * 5,
            "clocks": clocks}))
    if dist is not None:
        dist.destroy_process_group()
    return 0


# ---------------------------------------------------------------------------
# Single-layer workloads (`--workload wtconv1d | segmentation | train`): the other BASELINE layer
# configurations and the layer-set training step as lines of their own (1 GPU; also the small
# cases the profiler captures run, with --batch)
# ---------------------------------------------------------------------------
def run_single(args):
    import wtconv_b200
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the WTConv kernels have no CPU path")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    timer = Timer(dev, None)
    peak, peak_kind = load_peaks()
    sampler = ClockSampler(dev.index)
    sampler.start()
    kind = args.workload
    if kind == "wtconv1d":
        B = args.batch if args.batch != 128 else 512
        C, L, N = 64, 4, args.length
        m = load_state(wtconv_b200.WTConv1d(C, C, kernel_size=KSIZE, wt_levels=L), synthetic_state(C, L, 500, ndim=1)).to(dev).eval()
        nb = max(2, min(4, int(1.2e9 / (B * C * N * 4))))
        xs = [torch.randn(B, C, N, device=dev) for _ in range(nb)]
        nbytes = 2 * B * C * N * 4 + param_bytes(C, L, 4, ndim=1)
        name, dtype, launches = f"WTConv1d(64,64,5,wt_levels=4) on ({B},64,{N}) fp32", "f32", 1
        metric = "wtconv1d_layer_algorithmic_GBps"
    elif kind == "segmentation":
        B = args.batch if args.batch != 128 else 2
        C, L, H = 256, 5, 512
        m = load_state(wtconv_b200.WTConv2d(C, C, kernel_size=KSIZE, wt_levels=L), synthetic_state(C, L, 400)).to(dev).to(torch.bfloat16).eval()
        xs = [torch.randn(B, C, H, H, device=dev, dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last) for _ in range(2)]
        nbytes = layer_bytes(B, C, H, L, 2)
        name, dtype, launches = f"WTConv2d(256,256,5,wt_levels=5) on ({B},256,512,512) bf16 channels-last", "bf16", layer_launches(B, C, H, L)
        metric = "wtconv2d_segmentation_layer_algorithmic_GBps"
    else:   # train: forward + backward (input and parameter gradients) of the four stage layers, bf16
        B = args.batch
        layers = [l.train() for l in build_layers(dev)]
        for l in layers:
            for q in l.parameters():
                q.requires_grad_(True)
            l.wt_filter.requires_grad_(False)
            l.iwt_filter.requires_grad_(False)
        xs = [[torch.randn(B, C, H, H, device=dev, dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last).requires_grad_(True)
               for C, H, L in STAGES] for _ in range(2)]
        gs = [torch.randn_like(x) for x in xs[0]]
        nbytes = 3 * step_bytes(B)       # x, dL/dy read and dL/dx written on top of the forward's traffic, roughly
        name, dtype, launches = f"layer set forward + backward at batch {B}, bf16 channels-last", "bf16", None
        metric = "wtconv2d_layer_set_train_step_ms"

    if kind == "train":
        def step(i):
            for l, x, g in zip(layers, xs[i % 2], gs):
                l.zero_grad(set_to_none=True)
                x.grad = None
                l(x).backward(g)
        per = []
        for w in range(max(3, args.windows // 5)):
            for i in range(args.warmup if w == 0 else 0):
                step(i)
            per.append(timer.window(step, max(2, args.steps // 4)))
    else:
        per = timer.run(lambda i: m(xs[i % len(xs)]), args.steps, args.warmup, max(3, args.windows // 5))
    ms = statistics.median(per)
    clocks = sampler.stop()
    gbps = nbytes / (ms * 1e-3) / 1e9
    line = {"metric": metric, "value": ms if kind == "train" else gbps, "unit": "ms" if kind == "train" else UNIT, "n_gpus": 1,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": kind != "train",
            "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": {"workload": name},
            "roofline": None if kind == "train" else {"bound": "hbm", "achieved": gbps, "peak": peak, "unit": "GB/s",
                                                      "frac": gbps / peak, "traffic": None, "peak_source": f"of {peak_kind}"},
            "cpu_baseline": None, "e2e": None, "gpu_launches": None if launches is None else launches * args.steps * max(3, args.windows // 5),
            "clocks": clocks}
    print(json.dumps(line))
    return 0


def main():
    global BATCH, STAGES, WINDOWS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=128, help="per-GPU batch (128 = the BASELINE workload; "
                    "smaller values are for profiler captures)")
    ap.add_argument("--stages", default="0,1,2,3", help="subset of the four stage layers (profiler captures)")
    ap.add_argument("--workload", default="layers", choices=["layers", "model", "wtconv1d", "segmentation", "train"],
                    help="layers: the WTConv2d layer set (headline); model: WTConvNeXt-T images/sec; wtconv1d / "
                         "segmentation: the 1-D and the 512x512 layer alone; train: forward + backward of the layer set")
    ap.add_argument("--length", type=int, default=4096, help="signal length of --workload wtconv1d")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary measurements (profiler captures)")
    ap.add_argument("--windows", type=int, default=WINDOWS, help="timed windows of --steps steps (median reported)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    if args.workload == "model":
        return run_model(args)
    if args.workload in ("wtconv1d", "segmentation", "train"):
        WINDOWS = max(1, args.windows)
        args.windows = WINDOWS
        if args.workload == "train":
            BATCH = args.batch
            STAGES = [STAGES[int(i)] for i in args.stages.split(",")]
        return run_single(args)
    BATCH = args.batch
    WINDOWS = max(1, args.windows)
    STAGES = [STAGES[int(i)] for i in args.stages.split(",")]
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
