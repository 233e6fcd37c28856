#!/usr/bin/env python
"""Benchmark of the CATS sparse-MLP decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl cats|reference]
                    [--workload mistral7b|llama7b|llama70b] [--layers L] [--sparsity S] [--batch B]

One *step* is one decoded token through a stack of L CATS MLP layers (distinct weights per layer,
residual add + RMS norm between layers), i.e. the MLP half of a decoder's per-token work.  The
default workload is the Mistral-7B MLP stack: 32 layers, hidden 4096, intermediate 14336, fp16,
50 % sparsity, batch 1 (thresholds calibrated on 256 seeded vectors; weights N(0, 0.02^2); all
data synthetic).  Metric: decode tokens/s of that stack (and us/layer = step time / L).

Numbers in the JSON line:
  value        device-resident: state already in HBM, K steps timed with CUDA events
  e2e          through CatsMLPStack.decode_step: pinned host input -> H2D -> all layers -> D2H
  roofline     dominant kernel: algorithmic bytes per launch / mean launch duration (CUDA events
               around single launches, rotating over the layers so nothing is L2-resident)
  cpu_baseline the reference's dense thresholded PyTorch MLP on this host's cores (bounded sample)

With --impl reference only the CPU arm runs (rank 0 only under torchrun).
With N > 1 (torchrun) the stack is sharded along the intermediate dimension, one all-reduce per
layer; timing is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOADS = {
    # name: (shape key, dtype, layers, sparsity)
    "mistral7b": ("mistral7b", torch.float16, 32, 0.5),
    "llama7b": ("llama7b", torch.float16, 32, 0.5),
    "llama7b_fp32": ("llama7b", torch.float32, 32, 0.5),
    "llama70b": ("llama70b", torch.bfloat16, 80, 0.7),
}
# dram__bytes_read + dram__bytes_write per layer of k_cats_mega for the default workload, from the
# ncu capture summarised in profiles/k_cats_mega_mistral7b_fp16_s50_ncu_full.md (2 layers captured;
# traffic is proportional to the number of layers)
NCU_TRAFFIC_PER_LAYER = {("mistral7b", 0.5, 1): 236.7e6}
METRIC = "cats_mlp_stack_decode_tokens_per_s"
UNIT = "tokens/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="cats", choices=["cats", "reference"])
    ap.add_argument("--workload", default="mistral7b", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--sparsity", type=float, default=-1.0)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-sample-layers", type=int, default=4)
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-dense", action="store_true")
    ap.add_argument("--tp", default="fused", choices=["fused", "nccl"],
                    help="N > 1: exchange inside the persistent kernel, or one NCCL all-reduce per layer")
    return ap.parse_args()


def workload_config(args):
    shape, dtype, layers, sparsity = WORKLOADS[args.workload]
    from cats_b200 import synth

    H, I = synth.SHAPES[shape]
    L = args.layers or layers
    s = sparsity if args.sparsity < 0 else args.sparsity
    return H, I, dtype, L, s


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self.power = [], set(), None, []
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            uuid = torch.cuda.get_device_properties(index).uuid
            self.h = None
            for i in range(pynvml.nvmlDeviceGetCount()):
                h = pynvml.nvmlDeviceGetHandleByIndex(i)
                u = pynvml.nvmlDeviceGetUUID(h)
                u = u.decode() if isinstance(u, bytes) else u
                if str(uuid) in u:
                    self.h = h
            if self.h is None:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples),
                "power_w_max": max(self.power) if self.power else None}


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's dense thresholded MLP on the host cores
# ---------------------------------------------------------------------------------------------
def cpu_layers(H, I, n_layers, sparsity, seed):
    """fp32 CPU copies of ``n_layers`` layers (16-bit workloads are upcast: the reference's CPU
    path computes in fp32) with thresholds calibrated like the GPU arm's."""
    from cats_b200 import synth

    layers = []
    for l in range(n_layers):
        layer = synth.make_layer(H, I, torch.float32, torch.device("cpu"), seed * 1000 + l, sparsity)
        layers.append((layer.wg, layer.wu, layer.wdt.t().contiguous(), layer.threshold))
    return layers


def cpu_step(layers, x):
    """One pass over the sample layers with the same residual + RMS norm chaining."""
    from oracle.cats_oracle import torch_dense_masked_mlp

    r = x.clone()
    for wg, wu, wd, thr in layers:
        y = torch_dense_masked_mlp(x, wg, wu, wd, thr)
        r = r + y
        x = r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + 1e-6)
    return x


def time_cpu(H, I, L, sparsity, batch, seed, sample_layers, seconds=None, steps=None, warmup=3):
    from cats_b200 import synth

    torch.set_num_threads(os.cpu_count() or 1)
    n = min(sample_layers, L)
    layers = cpu_layers(H, I, n, sparsity, seed)
    x = synth.make_x(batch, H, torch.float32, torch.device("cpu"), seed + 5).reshape(batch, 1, H)
    with torch.no_grad():
        for _ in range(warmup):
            cpu_step(layers, x)
        times = []
        t_end = time.perf_counter() + (seconds or 1e9)
        while True:
            t0 = time.perf_counter()
            cpu_step(layers, x)
            times.append(time.perf_counter() - t0)
            if steps is not None and len(times) >= steps:
                break
            if steps is None and time.perf_counter() > t_end:
                break
    per_layer = statistics.mean(times) / n
    return {"per_layer_s": per_layer, "passes": len(times), "layers": n,
            "cores": torch.get_num_threads(), "step_s": per_layer * L}


def cpu_baseline_block(res, L, H, I, batch):
    return {"value": 1.0 / res["step_s"], "unit": UNIT, "cores": res["cores"], "kind": "port",
            "us_per_layer": res["per_layer_s"] * 1e6,
            "sample": (f"{res['passes']} passes over {res['layers']} of the {L} layers "
                       f"(H {H}, I {I}, batch {batch}, fp32 on CPU), dense thresholded PyTorch MLP "
                       f"(oracle/cats_oracle.py:torch_dense_masked_mlp), scaled to {L} layers")}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    H, I, dtype, L, s = workload_config(args)
    res = time_cpu(H, I, L, s, args.batch, args.seed, args.cpu_sample_layers,
                   steps=max(1, args.steps), warmup=max(1, args.warmup))
    value = 1.0 / res["step_s"]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": res["step_s"] * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_block(args, H, I, dtype, L, s, 1),
        "cpu_baseline": cpu_baseline_block(res, L, H, I, args.batch),
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def config_block(args, H, I, dtype, L, s, world):
    return {
        "workload": (f"{args.workload} CATS MLP stack: {L} layers, hidden {H}, intermediate {I}, "
                     f"{str(dtype).replace('torch.', '')}, sparsity {s}, batch {args.batch}, decode"),
        "layers": L, "hidden": H, "intermediate": I, "sparsity": s, "batch": args.batch,
        "parallelism": "single GPU" if world == 1 else f"tp{world} over the intermediate dimension, "
                                                       "one exchange of partial sums per layer",
        "l2": "inputs larger than L2: every step streams the distinct weights of all layers "
              "(GBs) once, nothing is reused between layers or steps",
        "seed": args.seed,
    }


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def event_time_ms(fn, iters, stream):
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(stream)
    for _ in range(iters):
        fn()
    e.record(stream)
    e.synchronize()
    return s.elapsed_time(e) / iters


def per_launch_us(launch_one, n_items, repeats, stream):
    """Mean duration of single launches, each bracketed by its own pair of CUDA events."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(n_items * repeats)]
    k = 0
    for _ in range(repeats):
        for i in range(n_items):
            evs[k][0].record(stream)
            launch_one(i)
            evs[k][1].record(stream)
            k += 1
    torch.cuda.synchronize()
    ts = [a.elapsed_time(b) * 1e3 for a, b in evs]
    return statistics.mean(ts), statistics.median(ts), min(ts)


def run_gpu_arm(args):
    import torch.distributed as dist

    from cats_b200 import _lib, ops, synth, tp
    from cats_b200.stack import CatsMLPStack

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py --impl cats needs a CUDA device (no CPU fallback)")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    H, I, dtype, L, s = workload_config(args)
    B = args.batch
    esize = torch.empty((), dtype=dtype).element_size()

    # ---- data: full layers are generated one at a time and sharded at once (TP) -------------
    layers = []
    for l in range(L):
        layer = synth.make_layer(H, I, dtype, dev, args.seed * 1000 + l, s)
        if world > 1:
            layer = tp.shard_layer(layer, rank, world)
        layers.append(layer)
    torch.cuda.synchronize()
    I_local = layers[0].wg.shape[0]
    x0 = synth.make_x(B, H, dtype, dev, args.seed + 5).reshape(B, H)
    stream = torch.cuda.current_stream(dev)

    if world == 1:
        stack = CatsMLPStack(layers, batch=B)
        stack.x_host.copy_(x0.cpu())
        run = stack.run_device
    else:
        # product path: one persistent kernel per GPU exchanging partial sums over NVLink itself;
        # the kernels + NCCL all-reduce graph only if that cannot be set up on every rank
        tp_mode, why = "fused", ""
        stack = None
        if args.tp == "fused":
            try:
                stack = tp.FusedTPStack(layers, batch=B)
                stack.set_input(x0)
                stack.run_device()
                torch.cuda.synchronize()
                if stack.device_status() != 0:
                    raise RuntimeError("device status %d" % stack.device_status())
            except Exception as e:  # noqa: BLE001 - reported in the JSON line
                why, stack = f"{type(e).__name__}: {e}"[:200], None
            okf = torch.tensor([1 if stack is not None else 0], device=dev)
            dist.all_reduce(okf, op=dist.ReduceOp.MIN)
            if int(okf.item()) == 0:
                stack = None
        if stack is None:
            tp_mode = "nccl" if args.tp == "nccl" else f"nccl (fused unavailable: {why or 'on another rank'})"
            stack = tp.TPStack(layers, batch=B)
            stack.set_input(x0)
            stack.capture()
        run = stack.run_device
        x_host = x0.cpu().pin_memory()
        out_host = torch.empty_like(x_host).pin_memory()
    stack.set_input(x0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ---------------------------------------------------------------
    for _ in range(max(3, args.warmup)):
        run()
    barrier()
    with ClockSampler(local_rank) as clocks:
        ms = event_time_ms(run, args.steps, stream)
        barrier()
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item())

    # ---- end to end through the host-buffer entry point ------------------------------------
    if world == 1:
        def e2e_step():
            stack.decode_step()
        h2d, d2h = stack.h2d_bytes, stack.d2h_bytes
    else:
        def e2e_step():
            stack.set_input(x_host)
            stack.run_device()
            out_host.copy_(stack.x, non_blocking=True)
            stream.synchronize()
        h2d = d2h = x_host.numel() * x_host.element_size()
    for _ in range(3):
        e2e_step()
    barrier()
    ms_e2e = event_time_ms(e2e_step, args.steps, stream)
    barrier()
    t = torch.tensor([ms_e2e], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_e2e = float(t.item())

    # ---- roofline of the kernel that ran in the timed region ------------------------------------
    # Algorithmic bytes of one layer: all of Wg, the active rows of Wu and WdT, x in, out.
    ws = stack.ws
    xin = x0.reshape(B, 1, H).clone()
    out = torch.empty_like(xin)
    if world == 1:
        stack.set_input(x0)
        counts = stack.active_counts()
    else:
        counts = []
        for l in layers[: min(L, 8)]:
            ops.gate(xin, l.wg, l.threshold, ws=ws)
            counts.append(ws.counters()[0])
    n_act = statistics.mean(counts)
    bytes_gate = esize * I_local * H + esize * B * H
    bytes_updown = 2 * esize * n_act * H + 2 * esize * B * H
    bytes_layer = bytes_gate + bytes_updown
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    us_layer = ms_step * 1e3 / L
    if world == 1:
        mega = _lib.lib().cats_uses_persistent_kernel(L, B, H, I_local, ops.dtype_code(dtype)) == 1
    else:
        mega = isinstance(stack, tp.FusedTPStack)
        if mega and stack.device_status() != 0:
            raise RuntimeError("a bounded wait ran out inside the tensor-parallel kernel")
    # tensor parallel: the all-reduce variant timed beside the fused kernel (context)
    nccl_variant = None
    if world > 1 and mega and not args.no_dense:
        ref_stack = tp.TPStack(layers, batch=B)
        ref_stack.set_input(x0)
        ref_stack.capture()
        for _ in range(3):
            ref_stack.run_device()
        barrier()
        ms_ref = event_time_ms(ref_stack.run_device, max(5, args.steps // 4), stream)
        barrier()
        t = torch.tensor([ms_ref], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        nccl_variant = {"us_per_layer": float(t.item()) * 1e3 / L,
                        "what": "stage kernels + one NCCL all-reduce + tail per layer, CUDA graph",
                        "speedup_of_fused": float(t.item()) / ms_step}
    # the two staged kernels on their own (single launches bracketed by events, rotating over the
    # layers): what a caller of the stage-level entry points gets, and the pre-fusion baseline
    reps = max(1, min(10, 320 // L))
    gate_us = per_launch_us(lambda i: ops.gate(xin, layers[i].wg, layers[i].threshold, ws=ws),
                            L, reps, stream)
    ops.gate(xin, layers[0].wg, layers[0].threshold, ws=ws)
    updown_us = per_launch_us(lambda i: ops.updown(xin, layers[i].wu, layers[i].wdt, ws, out=out),
                              L, reps, stream)
    staged = {
        "k_gate_tma": {"us": gate_us[0], "bytes": bytes_gate, "GBps": bytes_gate / gate_us[0] / 1e3},
        "k_updown_tma": {"us": updown_us[0], "bytes": bytes_updown,
                         "GBps": bytes_updown / updown_us[0] / 1e3},
    }
    if mega:
        # one launch of the persistent kernel = one step = L layers
        kname, launch_us, launch_bytes = "k_cats_mega", ms_step * 1e3, bytes_layer * L
    else:
        kname = max(staged, key=lambda k: staged[k]["us"])
        launch_us, launch_bytes = staged[kname]["us"], staged[kname]["bytes"]
    achieved = launch_bytes / launch_us / 1e3
    roofline = {
        "bound": "hbm", "kernel": kname, "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak, "peak_source": peak_src,
        "traffic": (NCU_TRAFFIC_PER_LAYER[(args.workload, s, B)] * L
                    if mega and (args.workload, s, B) in NCU_TRAFFIC_PER_LAYER else None),
        "bytes_per_launch": launch_bytes, "launch_us": launch_us,
        "units_per_launch": f"{L} layers" if mega else "1 layer stage",
        "frac_of_8TBps_nominal": achieved / 8000.0,
        "layer": {"bytes": bytes_layer, "us": us_layer, "GBps": bytes_layer / us_layer / 1e3,
                  "frac": bytes_layer / us_layer / 1e3 / peak,
                  "frac_of_8TBps": bytes_layer / us_layer / 1e3 / 8000.0},
        "staged_kernels": staged, "n_active_mean": n_act, "intermediate_local": I_local,
    }

    # ---- statistics kernel beside the path (threshold calibration): HBM-bound stream ----------
    stats = None
    if world == 1 and not args.no_dense:
        nval = 160 * 1000 * 1000                       # 320 MB of fp16 activations: larger than L2
        vals = torch.nn.functional.silu(torch.randn(nval // 8, device=dev) * 1.28).to(dtype).repeat(8)
        edges = torch.cat([torch.tensor([-torch.inf]), torch.linspace(-1, 1, 998),
                           torch.tensor([torch.inf])]).to(dev)
        hcounts = torch.zeros(999, dtype=torch.int64, device=dev)
        for _ in range(2):
            ops.histogram(vals, edges, hcounts, take_abs=True)
        h_us = per_launch_us(lambda i: ops.histogram(vals, edges, hcounts, take_abs=True), 1, 5, stream)
        hb = vals.numel() * vals.element_size()
        stats = {"k_histogram": {"us": h_us[1], "bytes": hb, "GBps": hb / h_us[1] / 1e3,
                                 "frac": hb / h_us[1] / 1e3 / peak,
                                 "bound": "instruction issue (about 20 instructions per value), not HBM",
                                 "what": f"|post-activation| histogram of {vals.numel()} {dtype} values "
                                         "(SiLU of N(0, 1.28^2)), the reference's 999 bins"}}
        del vals

    # ---- dense cuBLAS MLP of the same shape (context; single GPU only) -----------------------
    dense = None
    if world == 1 and not args.no_dense:
        import torch.nn.functional as F

        xs = x0.reshape(B, 1, H).clone()
        wds = [l.wdt.t() for l in layers]

        def dense_step():
            xx, r = xs, xs
            for l, wd in zip(layers, wds):
                y = F.linear(F.silu(F.linear(xx, l.wg)) * F.linear(xx, l.wu), l.wdt.t())
                r = r + y
                xx = (r.float() * torch.rsqrt(r.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(dtype)
            return xx

        g = torch.cuda.CUDAGraph()
        sside = torch.cuda.Stream(dev)
        sside.wait_stream(stream)
        with torch.cuda.stream(sside):
            for _ in range(2):
                dense_step()
        stream.wait_stream(sside)
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            dense_step()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        ms_dense = event_time_ms(g.replay, max(5, args.steps // 4), stream)
        dense = {"us_per_layer": ms_dense * 1e3 / L, "tokens_per_s": 1e3 / ms_dense,
                 "what": "torch F.linear x3 + SiLU*mul + residual/RMS-norm per layer, CUDA graph",
                 "speedup_of_cats": ms_dense / ms_step}

    def leave():
        """Multi-rank exit: a last barrier, then leave without tearing NCCL down — destroying the
        process group while a captured CUDA graph still references its collectives can block."""
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier()
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)

    if rank != 0:
        leave()
        return

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        res = time_cpu(H, I, L, s, B, args.seed, args.cpu_sample_layers, seconds=args.cpu_seconds)
        cpu = cpu_baseline_block(res, L, H, I, B)

    line = {
        "metric": METRIC, "value": 1e3 / ms_step, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
        "us_per_layer": us_layer, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": {torch.float16: "f16", torch.bfloat16: "bf16",
                                       torch.float32: "f32"}[dtype] + " storage, f32 accumulate",
        "data": "synthetic", "config": config_block(args, H, I, dtype, L, s, world),
        "e2e": {"value": 1e3 / ms_e2e, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "api": "CatsMLPStack.decode_step (pinned host in/out, cats_mlp_stack C call)"
                if world == 1 else ("FusedTPStack (pinned host in/out, one cats_tp_mlp_stack C call per rank)"
                                    if mega else "TPStack (CUDA graph of kernels + NCCL all-reduce)")},
        "gpu_launches": args.steps * (1 if mega else stack.launches_per_step),
        "roofline": roofline, "clocks": clocks.summary(), "dense_cublas": dense,
        "cpu_baseline": cpu,
    }
    if stats is not None:
        line["roofline"]["stats_kernels"] = stats
    if world > 1:
        line["tp"] = {"mode": tp_mode, "nccl_allreduce_variant": nccl_variant}
    emit(line)
    leave()


_RESULT_FD = None


def claim_stdout():
    """Keep stdout for the one JSON line: whatever libraries print on file descriptor 1 from now
    on (NCCL writes its version line there) goes to stderr instead."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        sys.stdout.flush()
        os.write(_RESULT_FD, data)


def main():
    args = parse_args()
    claim_stdout()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
