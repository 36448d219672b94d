#!/usr/bin/env python
"""Benchmark of the WTConv2d forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the BASELINE layer set): the four WTConvNeXt-T stage layers
WTConv2d(C,C,kernel_size=5,wt_levels=L) with (C,H=W,L) = (96,56,5), (192,28,4),
(384,14,3), (768,7,2), batch 128 per GPU, bf16, channels-last, x ~ N(0,1), seeded
random weights with wavelet_scale ~ U(0.05,0.2).  A "step" is one forward pass of
all four layers.  The metric is algorithmic bytes (input + output + parameters,
intermediates count zero) per second, in GB/s, summed over all ranks.

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the
reference forward (oracle/wtconv_torch.py: the same ATen operator sequence as the
reference modules, which cannot travel to the GPU box) on the host cores.
"""
from __future__ import annotations

import argparse
import json
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
METRIC = "wtconv2d_layer_set_algorithmic_GBps"
UNIT = "GB/s"


def param_bytes(C, L, elem):
    # (C*K^2 + C bias + C base_scale + L*(4C*K^2 + 4C)) * sizeof(param)
    return (C * KSIZE * KSIZE + C + C + L * (4 * C * KSIZE * KSIZE + 4 * C)) * elem


def layer_bytes(B, C, H, L, elem):
    return 2 * B * C * H * H * elem + param_bytes(C, L, elem)


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


def make_params(stage, dtype):
    from oracle import wtconv_torch           # seeded synthetic parameters (shapes of the reference layer)
    C, H, L = STAGES[stage]
    return wtconv_torch.random_params(C, KSIZE, L, seed=100 + stage, dtype=dtype)


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
# CPU arm: the oracle port of the reference forward on the host cores
# ---------------------------------------------------------------------------
def cpu_layer_set_seconds(batch, reps, threads):
    """Seconds per pass of the four stage layers at `batch`, fp32 channels-last (the reference's
    fastest CPU form), with `threads` host threads.  Returns the median over `reps` passes."""
    from oracle import wtconv_torch
    torch.set_num_threads(threads)
    layers = []
    for si, (C, H, L) in enumerate(STAGES):
        params = make_params(si, torch.float32)
        g = torch.Generator().manual_seed(300 + si)
        x = torch.randn(batch, C, H, H, generator=g).contiguous(memory_format=torch.channels_last)
        layers.append((x, params))
    times = []
    with torch.no_grad():
        for rep in range(reps + 1):
            t0 = time.perf_counter()
            for x, params in layers:
                wtconv_torch.wtconv2d_forward(x, params)
            if rep > 0:                       # first pass is the warm-up
                times.append(time.perf_counter() - t0)
    return statistics.median(times)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = os.cpu_count() or 1
    batch = 32                                 # bounded sample: a quarter of the per-GPU batch per step
    secs = []
    for _ in range(args.warmup):
        cpu_layer_set_seconds(batch, 1, threads)
    for _ in range(args.steps):
        secs.append(cpu_layer_set_seconds(batch, 1, threads))
    t = statistics.median(secs)
    value = step_bytes(batch) / t / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "WTConvNeXt-T layer set (4 stage shapes), K=5, channels-last", "batch_per_step": batch,
                   "note": "CPU restatement of the reference forward (same ATen operator sequence); bytes counted "
                           "at the workload's bf16 element size so that the ratio to the GPU arm is a speed ratio"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"layer set at batch {batch} (1/4 of the per-GPU batch), fp32 channels-last, "
                                   f"median of {args.steps} passes"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def build_layers(dev):
    import wtconv_b200
    layers = []
    for si, (C, H, L) in enumerate(STAGES):
        m = wtconv_b200.WTConv2d(C, C, kernel_size=KSIZE, wt_levels=L, bias=True)
        sd = m.state_dict()
        for k, v in make_params(si, torch.float32).items():
            sd[k] = v.reshape(sd[k].shape)
        m.load_state_dict(sd, strict=True)
        layers.append(m.to(dev).to(torch.bfloat16).eval())
    return layers


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

    layers = build_layers(dev)
    nsets = 2                                      # rotating input sets: 2 x 289 MB of traffic between reuses
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    host_in = [[torch.randn(BATCH, C, H, H, generator=g).to(torch.bfloat16)
                .contiguous(memory_format=torch.channels_last).pin_memory() for C, H, L in STAGES]
               for _ in range(1)]
    dev_in = [[t.to(dev, non_blocking=True) for t in host_in[0]] for _ in range(nsets)]
    host_out = [torch.empty_like(t).pin_memory() for t in host_in[0]]
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def step(i):
        outs = []
        for m, x in zip(layers, dev_in[i % nsets]):
            outs.append(m(x))
        return outs

    def timed(fn, steps, warmup, join=None):
        with torch.no_grad():
            for i in range(warmup):
                fn(i)
            if join is not None:
                join()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(steps):
                fn(i)
            if join is not None:
                join()                      # side streams rejoin the timed stream before the end event
            e1.record()
            barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            from wtconv_b200.sharding import max_over_ranks
            ms = max_over_ranks(ms, dev)
        return ms / steps

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step = timed(step, args.steps, args.warmup)

    # end to end through the public modules with HOST buffers: pinned host -> device copy of the
    # four inputs, the four forwards, device -> pinned host copy of the four outputs, every step
    # The three legs run on three streams (as a serving loop would): the upload of step i+1 and the
    # download of step i-1 overlap the kernels of step i; every step still moves all its bytes.
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    bufs = [[torch.empty_like(t, device=dev) for t in host_in[0]] for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        k = i % 2
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_cmp[k])              # the kernels that last read bufs[k] are done
            for d, h in zip(bufs[k], host_in[0]):
                d.copy_(h, non_blocking=True)
            ev_in[k].record(s_in)
        main.wait_event(ev_in[k])
        outs = [m(x) for m, x in zip(layers, bufs[k])]
        ev_cmp[k].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp[k])
            for ho, yv in zip(host_out, outs):
                ho.copy_(yv, non_blocking=True)
                yv.record_stream(s_out)

    def e2e_join():
        main.wait_stream(s_in)
        main.wait_stream(s_out)
    ms_e2e = timed(e2e_step, max(4, args.steps // 2), 2, e2e_join)

    # dominant launch: the stage-1 layer (C=96, 56x56, 5 levels), timed alone on rotating inputs
    x1 = [dev_in[k][0] for k in range(nsets)] + [torch.randn_like(dev_in[0][0]) for _ in range(2)]
    ms_l1 = timed(lambda i: layers[0](x1[i % len(x1)]), max(args.steps, 10), 3)
    clocks = sampler.stop() if rank == 0 else None

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
    in_bytes = sum(t.numel() * t.element_size() for t in host_in[0])
    cpu = None
    if world == 1 or rank == 0:
        threads = os.cpu_count() or 1
        sample_b = 32
        t_cpu = cpu_layer_set_seconds(sample_b, 3, threads)
        cpu = {"value": step_bytes(sample_b) / t_cpu / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"oracle port of the reference forward, layer set at batch {sample_b} "
                         f"(1/4 of the per-GPU batch), fp32 channels-last, median of 3 passes"}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "WTConvNeXt-T layer set: WTConv2d K=5, (C,H,L)=(96,56,5),(192,28,4),(384,14,3),"
                               "(768,7,2), batch 128 per GPU, bf16 storage, channels-last",
                   "io_dtype": "bf16", "cache": f"{nsets} rotating input sets, 289 MB of traffic per step (> L2)",
                   "sharding": "batch, no collective on the data path"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_source": f"of {peak_kind}",
                     "kernel": "stage-1 layer call (low-pass reduction, wt2d_regplane_kernel, wt2d_deep_kernel, "
                               "wt2d_final_kernel)",
                     "algorithmic_bytes_per_launch": l1_bytes, "ms_per_launch": ms_l1},
        "cpu_baseline": cpu,
        "e2e": {"value": total_bytes / (ms_e2e * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": in_bytes},
        "gpu_launches": sum(layer_launches(BATCH, C, H, L) for C, H, L in STAGES) * args.steps,
        "clocks": clocks,
    }
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


# ---------------------------------------------------------------------------
# Secondary workload: full WTConvNeXt-T inference (images/sec), `--workload model`
# ---------------------------------------------------------------------------
class _OracleLayer(torch.nn.Module):
    """CPU arm of the model workload: the layer's parameters with the oracle's operator sequence."""

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
    from wtconv_b200.wtconvnext_harness import CapturedForward, WTConvNeXtTiny
    torch.set_num_threads(threads)
    torch.manual_seed(0)
    model = WTConvNeXtTiny(_OracleLayer).eval()
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
    torch.manual_seed(0)
    model = WTConvNeXtTiny(wtconv_b200.WTConv2d).to(dev).to(torch.bfloat16).eval()
    model = model.to(memory_format=torch.channels_last)
    g = torch.Generator().manual_seed(77 + rank)
    host = [torch.randn(batch, 3, 224, 224, generator=g).to(torch.bfloat16)
            .contiguous(memory_format=torch.channels_last).pin_memory() for _ in range(2)]
    xs = [h.to(dev) for h in host]
    host_out = torch.empty(batch, 1000, dtype=torch.bfloat16).pin_memory()

    def timed(fn, steps, warmup):
        with torch.no_grad():
            for i in range(warmup):
                fn(i)
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(steps):
                fn(i)
            e1.record()
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            from wtconv_b200.sharding import max_over_ranks
            ms = max_over_ranks(ms, dev)
        return ms / steps

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # the whole forward is one CUDA graph; a step copies the batch into its input buffer and replays
    fwd = CapturedForward(model, xs[0])
    ms = timed(lambda i: fwd(xs[i % 2]), args.steps, args.warmup)
    ms_e2e = timed(lambda i: host_out.copy_(fwd(host[i % 2]), non_blocking=True), max(2, args.steps // 2), 2)
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
                                for d, (C, H, L) in zip((3, 3, 9, 3), STAGES)) * args.steps,
            "clocks": clocks}))
    if dist is not None:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=128, help="per-GPU batch (128 = the BASELINE workload; "
                    "smaller values are for profiler captures)")
    ap.add_argument("--stages", default="0,1,2,3", help="subset of the four stage layers (profiler captures)")
    ap.add_argument("--workload", default="layers", choices=["layers", "model"],
                    help="layers: the WTConv2d layer set (headline); model: WTConvNeXt-T images/sec")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    if args.workload == "model":
        return run_model(args)
    global BATCH, STAGES
    BATCH = args.batch
    STAGES = [STAGES[int(i)] for i in args.stages.split(",")]
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
