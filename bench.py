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
import math
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
# (dram__bytes_read + dram__bytes_write) / algorithmic bytes of k_cats_mega for the default
# workload, from the ncu capture summarised in profiles/k_cats_mega_mistral7b_fp16_s50_ncu_full.md
# (4 layers captured: 950.75 MB read + written against 943.95 MB algorithmic; DRAM traffic is the
# rows a rank streams, so it grows with the layers and with the rows per rank like the
# algorithmic bytes)
NCU_TRAFFIC_RATIO = {("mistral7b", 0.5, 1): 950.75e6 / 943.95e6}
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
    ap.add_argument("--regions", type=int, default=10,
                    help="timed regions of --steps steps each (the median is reported)")
    ap.add_argument("--config5-layers", type=int, default=80)
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-config5", action="store_true")
    ap.add_argument("--no-decoder", action="store_true")
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


def per_launch_us(launch_one, n_items, repeats, stream, before=None):
    """Durations of single launches, each bracketed by its own pair of CUDA events (``before``
    runs ahead of each start event, e.g. an L2 flush).  Returns (mean, median, min, geomean)."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(n_items * repeats)]
    k = 0
    for _ in range(repeats):
        for i in range(n_items):
            if before is not None:
                before()
            evs[k][0].record(stream)
            launch_one(i)
            evs[k][1].record(stream)
            k += 1
    torch.cuda.synchronize()
    ts = [a.elapsed_time(b) * 1e3 for a, b in evs]
    return (statistics.mean(ts), statistics.median(ts), min(ts),
            math.exp(statistics.mean(math.log(max(t, 1e-3)) for t in ts)))


def graph_launch_us(launch_one, n_items, repeats, stream):
    """Mean duration of one launch when ``n_items`` launches (one per layer, so every launch reads
    weights that are not in L2) replay back to back from a CUDA graph: what the kernel takes when
    the host is not the limit (a Python call per launch costs as much as these kernels run).
    Returns a 1-tuple to read like per_launch_us()[0]."""
    launch_one(0)
    stream.synchronize()
    side = torch.cuda.Stream()             # capture needs a stream other than the default one
    side.wait_stream(stream)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for i in range(n_items):
            launch_one(i)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(side):
        g.replay()
        side.synchronize()
        e0.record(side)
        for _ in range(repeats):
            g.replay()
        e1.record(side)
    side.synchronize()
    return (e0.elapsed_time(e1) * 1e3 / (repeats * n_items),)


class Dist:
    """The process group of this run (or none), with the two operations the bench needs."""

    def __init__(self):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dev = torch.device("cuda", self.local_rank)

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        import torch.distributed as dist
        t = torch.tensor([v], device=self.dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())


def timed_regions(run, steps, regions, D: Dist, stream):
    """``regions`` timed regions of exactly ``steps`` steps each: barrier + synchronize on both
    sides, CUDA events on the launching stream, the maximum over ranks per region.  Returns the
    per-step times in ms, one per region."""
    out = []
    for _ in range(regions):
        D.barrier()
        ms = event_time_ms(run, steps, stream)
        D.barrier()
        out.append(D.max_over_ranks(ms))
    return out


def spread(samples):
    return {"median": statistics.median(samples), "min": min(samples), "max": max(samples),
            "n": len(samples)}


def hbm_peak():
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        return float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def make_layers(H, I, dtype, L, s, seed, D: Dist, keep_full=0):
    """L layers on the device, sharded over the intermediate dimension when there are several
    ranks (every rank generates the full layer from the seed and keeps its rows).  The first
    ``keep_full`` unsharded layers are returned as well (for the parity check)."""
    from cats_b200 import synth, tp

    layers, full = [], []
    for l in range(L):
        layer = synth.make_layer(H, I, dtype, D.dev, seed * 1000 + l, s)
        if l < keep_full:
            full.append(layer)
        layers.append(tp.shard_layer(layer, D.rank, D.world) if D.world > 1 else layer)
    torch.cuda.synchronize()
    return layers, full


def layer_bytes(layers, n_act, B, H, esize):
    I_local = layers[0].wg.shape[0]
    return esize * I_local * H + 2 * esize * n_act * H + 4 * esize * B * H


def chain_active_counts(stack, layers, B, H, limit=8):
    """Active neurons (union over the batch) of the first layers along the real chain: the layers
    one launch at a time from the stack's current input, with the counter read back after each.
    For reporting, outside every timed region."""
    from cats_b200 import ops

    counts = []
    x, r = stack.x.clone(), stack.resid.clone()
    nxt = torch.empty_like(x)
    for l in layers[:limit]:
        ops.mlp(x.reshape(B, 1, H), l.wg, l.wu, l.wdt, l.threshold, resid=r, x_next=nxt,
                eps=stack.eps, ws=stack.ws)
        counts.append(stack.ws.counters()[0])
        x, nxt = nxt, x
    return counts


def active_counts(layers, x0, B, H, ws, limit=8):
    """Active neurons (union over the batch) of the first layers for the input x0: stage 1 alone
    plus the counter read-back.  For reporting, outside every timed region."""
    from cats_b200 import ops

    xin = x0.reshape(B, 1, H).contiguous()
    counts = []
    for l in layers[:limit]:
        ops.gate(xin, l.wg, l.threshold, ws=ws)
        counts.append(ws.counters()[0])
    return counts


def parity_block(full, x0, B, H, dtype, D: Dist, tol):
    """The first layers through the product path against the CPU oracle of the UNSHARDED stack
    (the checker; rank 0 computes it), and, with several ranks, bit-identity of the result across
    ranks.  Raises outside the tolerance."""
    import numpy as np

    from cats_b200 import tp
    from cats_b200.stack import CatsMLPStack
    from oracle import cats_oracle as O

    sub = [tp.shard_layer(l, D.rank, D.world) for l in full] if D.world > 1 else full
    stack = tp.FusedTPStack(sub, batch=B) if D.world > 1 else CatsMLPStack(sub, batch=B)
    for _ in range(2):                        # twice: the exchange slots alternate across launches
        stack.set_input(x0)
        stack.run_device()
    torch.cuda.synchronize()
    status = stack.ws.counters()[1]
    same = True
    if D.world > 1:
        import torch.distributed as dist
        for t in (stack.x, stack.resid):
            parts = [torch.empty_like(t) for _ in range(D.world)]
            dist.all_gather(parts, t)
            same = same and all(torch.equal(parts[0], p) for p in parts)
    block = None
    if D.rank == 0:
        f = lambda t: t.detach().float().cpu().numpy()
        bf16 = lambda a: torch.from_numpy(np.asarray(a, np.float32)).to(torch.bfloat16).float().numpy()
        rnd = {torch.float16: np.float16, torch.float32: None, torch.bfloat16: bf16}[dtype]
        xe, re_, _ = O.mlp_stack(f(x0), [(f(l.wg), f(l.wu), f(l.wdt).T) for l in full],
                                 [l.threshold for l in full], round_to=rnd)
        block = {"layers": len(full), "rel_l2_x": O.rel_l2(f(stack.x), xe),
                 "rel_l2_resid": O.rel_l2(f(stack.resid), re_), "tolerance": tol,
                 "identical_across_ranks": bool(same), "device_status": int(status),
                 "against": "CPU oracle of the unsharded stack (oracle/cats_oracle.py:mlp_stack)"}
    if D.world > 1:
        stack.close()
    ok = torch.tensor([1], device=D.dev)
    if D.rank == 0 and not (block["rel_l2_x"] <= tol and block["rel_l2_resid"] <= tol and same
                            and status == 0):
        ok.zero_()
    if D.world > 1:
        import torch.distributed as dist
        dist.broadcast(ok, 0)
    if int(ok.item()) == 0:
        if D.rank == 0:
            sys.stderr.write("PARITY FAILURE: " + json.dumps(block) + "\n")
        raise SystemExit(3)
    return block


def build_tp_stack(layers, B, x0, mode, D: Dist):
    """Several ranks: the fused stack (one persistent kernel per GPU, exchange inside), or the
    kernels + one NCCL all-reduce per layer in a CUDA graph."""
    import torch.distributed as dist

    from cats_b200 import tp

    stack, why = None, ""
    if mode == "fused":
        try:
            stack = tp.FusedTPStack(layers, batch=B)
            stack.set_input(x0)
            stack.run_device()
            torch.cuda.synchronize()
            stack.check()
        except Exception as e:  # noqa: BLE001 - reported in the JSON line
            why, stack = f"{type(e).__name__}: {e}"[:200], None
        okf = torch.tensor([1 if stack is not None else 0], device=D.dev)
        dist.all_reduce(okf, op=dist.ReduceOp.MIN)
        if int(okf.item()) == 0:
            stack = None
    if stack is not None:
        return stack, "fused"
    stack = tp.TPStack(layers, batch=B)
    stack.set_input(x0)
    stack.capture()
    return stack, ("nccl" if mode == "nccl" else f"nccl (fused unavailable: {why or 'on another rank'})")


def measure_stack(name, H, I, dtype, L, s, B, args, D: Dist, regions, with_nccl=True, parity_layers=0,
                  sample_clocks=False):
    """Build a stack of the given shape (sharded when there are several ranks), time it and
    return a result block: us/layer, tokens/s, achieved GB/s per rank against the HBM peak."""
    from cats_b200 import _lib, ops, synth, tp
    from cats_b200.stack import CatsMLPStack

    esize = torch.empty((), dtype=dtype).element_size()
    stream = torch.cuda.current_stream(D.dev)
    layers, full = make_layers(H, I, dtype, L, s, args.seed, D, keep_full=parity_layers)
    x0 = synth.make_x(B, H, dtype, D.dev, args.seed + 5).reshape(B, H)
    parity = None
    if parity_layers:
        tol = {torch.float32: 1e-3, torch.float16: 2e-2, torch.bfloat16: 5e-2}[dtype]
        parity = parity_block(full, x0, B, H, dtype, D, tol)
        del full
    if D.world == 1:
        stack, mode = CatsMLPStack(layers, batch=B, sparsity=s), "single GPU"
        persistent = stack.launches_per_step == 1
    else:
        stack, mode = build_tp_stack(layers, B, x0, args.tp, D)
        persistent = isinstance(stack, tp.FusedTPStack)
    def step():
        # every step decodes the same token state (two 8 KB device copies): the active sets are
        # then the calibrated ones at every step and n_active below is what the kernel streamed;
        # without the reset the residual would keep growing from step to step
        stack.set_input(x0)
        stack.run_device()

    for _ in range(max(3, args.warmup)):
        step()
    clocks = None
    if sample_clocks:      # SM clock and throttle reasons DURING the timed regions
        with ClockSampler(D.local_rank) as sampler:
            samples = timed_regions(step, args.steps, regions, D, stream)
        clocks = sampler.summary()
    else:
        samples = timed_regions(step, args.steps, regions, D, stream)
    ms = statistics.median(samples)
    if persistent and D.world > 1:
        stack.check()
    stack.set_input(x0)
    n_act = statistics.mean(chain_active_counts(stack, layers, B, H))
    by = layer_bytes(layers, n_act, B, H, esize)
    peak, peak_src = hbm_peak()
    us_layer = ms * 1e3 / L
    block = {
        "workload": f"{name}: {L} layers, hidden {H}, intermediate {I}, "
                    f"{str(dtype).replace('torch.', '')}, sparsity {s}, batch {B}",
        "mode": mode, "layers": L, "us_per_layer": us_layer, "tokens_per_s": B * 1e3 / ms,
        "ms_per_step": ms, "ms_per_step_samples": samples, "bytes_per_layer_per_rank": by,
        "GBps_per_rank": by / us_layer / 1e3, "frac_of_peak": by / us_layer / 1e3 / peak,
        "frac_of_8TBps": by / us_layer / 1e3 / 8000.0, "peak_source": peak_src,
        "n_active_mean_per_rank": n_act, "intermediate_local": layers[0].wg.shape[0],
        "kernel": "k_cats_mega" if persistent else "staged kernels",
    }
    if D.world == 1 and stack.dense:
        # dense tensor-core path: every row of the three matrices is streamed
        streamed = 3 * esize * layers[0].wg.shape[0] * H + 4 * esize * B * H
        block.update({"kernel": "k_dense_stack (tcgen05, one cooperative launch for the stack)",
                      "bytes_streamed_per_layer": streamed,
                      "GBps_streamed": streamed / us_layer / 1e3,
                      "frac_of_peak_streamed": streamed / us_layer / 1e3 / peak,
                      "note": "bytes_per_layer_per_rank / frac_of_peak count the union's bytes "
                              "(all of Wg + the union's rows of Wu and Wd), *_streamed all three "
                              "matrices, which is what this path reads"})
    if parity is not None:
        block["parity"] = parity
    if clocks is not None:
        block["clocks"] = clocks
    if D.world > 1 and persistent and with_nccl:
        ref = tp.TPStack(layers, batch=B)
        ref.set_input(x0)
        ref.capture()

        def ref_step():
            ref.set_input(x0)
            ref.run_device()

        for _ in range(3):
            ref_step()
        rs = timed_regions(ref_step, max(5, args.steps // 2), 3, D, stream)
        block["nccl_allreduce_variant"] = {
            "us_per_layer": statistics.median(rs) * 1e3 / L,
            "what": "stage kernels + one NCCL all-reduce + tail per layer, CUDA graph",
            "speedup_of_fused": statistics.median(rs) / ms}
    return block, stack, layers, x0


def single_layer_block(layers, x0, B, H, I, dtype, ws, stream, n_act, esize, peak):
    """What a decoder sees: ONE ``cats_mlp`` call per layer.  (a) back to back over the distinct
    layers' weights (nothing stays in L2), one event pair per call; (b) the reference's
    micro-benchmark protocol, flash_gemv/bench/utils.py:12-58: an L2 flush (zero_() of a 512 MB
    buffer) before every timed call, per-call events, geometric mean - plus the reference's
    "Optimal" column (flash_gemv/bench/profile_llama7B.py:66-69): the dense MLP with the
    intermediate dimension cut down to the active count."""
    import torch.nn.functional as F

    from cats_b200 import ops

    from cats_b200 import _lib

    L = len(layers)
    xin = x0.reshape(B, 1, H).contiguous()
    out = torch.empty_like(xin)
    call = lambda i: ops.mlp(xin, layers[i].wg, layers[i].wu, layers[i].wdt, layers[i].threshold,
                             out=out, ws=ws)
    by = esize * I * H + 2 * esize * n_act * H + 4 * esize * B * H
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=xin.device)
    row = lambda t: {"mean_us": t[0], "median_us": t[1], "min_us": t[2], "geomean_us": t[3]}
    dcode = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
    routes = {}
    # the two routes cats_mlp has for one token: the stage-1 / stage-2+3 kernel pair with
    # programmatic dependent launch (default) and a single-layer launch of the persistent kernel
    for name, pair in (("kernel_pair", 1), ("persistent_kernel", 0)):
        _lib.check(_lib.lib().cats_set_option(b"single_pair", pair))
        if name == "kernel_pair" and _lib.lib().cats_uses_persistent_kernel(1, B, H, I, dcode):
            continue                                   # this shape or batch has no pair route
        for i in range(min(L, 4)):
            call(i)
        b2b = per_launch_us(call, L, max(1, 128 // L), stream)
        gr = graph_launch_us(call, L, max(1, 128 // L), stream)
        fl = per_launch_us(call, L, max(1, 100 // L + 1), stream, before=flush.zero_)
        routes[name] = {
            "back_to_back": dict(row(b2b), GBps=by / b2b[1] / 1e3, frac_of_peak=by / b2b[1] / 1e3 / peak),
            "graph_replay_us": gr[0], "graph_replay_frac_of_peak": by / gr[0] / 1e3 / peak,
            "reference_protocol": row(fl)}
    _lib.check(_lib.lib().cats_set_option(b"single_pair", 1))
    default = "kernel_pair" if "kernel_pair" in routes else "persistent_kernel"
    fl = tuple(routes[default]["reference_protocol"][k] for k in ("mean_us", "median_us", "min_us", "geomean_us"))
    k = (int(round(n_act)) + 7) // 8 * 8      # whole 16-byte vectors of fp16, as cuBLAS likes them
    dense_call = lambda i: F.linear(F.silu(F.linear(xin, layers[i].wg)) * F.linear(xin, layers[i].wu),
                                    layers[i].wdt.t())
    opt_call = lambda i: F.linear(F.silu(F.linear(xin, layers[i].wg[:k])) * F.linear(xin, layers[i].wu[:k]),
                                  layers[i].wdt[:k].t())
    for i in range(2):
        dense_call(i), opt_call(i)
    dn = per_launch_us(dense_call, L, max(1, 100 // L + 1), stream, before=flush.zero_)
    op = per_launch_us(opt_call, L, max(1, 100 // L + 1), stream, before=flush.zero_)
    del flush
    return {
        "what": "one cats_mlp call per layer, both routes: back to back with an event pair per call, "
                "replayed from a CUDA graph of all layers (how a decoder runs it), and under the "
                "reference's micro-benchmark protocol",
        "default_route": default,
        "routes": routes,
        "back_to_back": routes[default]["back_to_back"],
        "reference_protocol": {
            "protocol": "L2 flush (512 MB zero_) before every call, per-call CUDA events, geometric "
                        "mean (flash_gemv/bench/utils.py:12-58)",
            "k_active": k, "cats": row(fl), "dense_cublas": row(dn),
            "optimal_dense_with_I_equal_k": row(op),
            "speedup_cats_over_dense_geomean": dn[3] / fl[3]},
    }


def sweep_block(args, D: Dist):
    """Other configurations on one GPU, a few layers each: the sparsity sweep of the Mistral
    shape, the Llama-2-7B shape in fp16 and fp32 (fp32 = the single-layer CPU configuration),
    and batches."""
    out = []
    cases = [("mistral7b", torch.float16, s, 1, 8) for s in (0.3, 0.7, 0.9)]
    cases += [("llama7b", torch.float16, 0.5, 1, 8), ("llama7b", torch.float32, 0.5, 1, 6)]
    cases += [("mistral7b", torch.float16, 0.5, b, 6) for b in (2, 4, 8, 16)]
    from cats_b200 import synth
    import torch.nn.functional as F

    for shape, dtype, s, B, L in cases:
        H, I = synth.SHAPES[shape]
        sub = argparse.Namespace(**vars(args))
        sub.steps, sub.warmup = max(10, args.steps // 2), 3
        block, stack, layers, x0 = measure_stack(shape, H, I, dtype, L, s, B, sub, D, regions=3,
                                                 with_nccl=False)
        if B > 1:   # the dense cuBLAS MLP at the same batch, same chaining, CUDA graph
            block["dense_cublas_us_per_layer"] = dense_stack_us(layers, x0, B, H, dtype, sub, D)
            block["speedup_of_cats"] = block["dense_cublas_us_per_layer"] / block["us_per_layer"]
        del block["ms_per_step_samples"]
        out.append(block)
        del stack, layers
        torch.cuda.empty_cache()
    return out


def dense_stack_us(layers, x0, B, H, dtype, args, D: Dist):
    """us/layer of the dense SiLU-gated MLP stack on cuBLAS (torch F.linear x3 + SiLU*mul +
    residual/RMS-norm per layer), replayed from a CUDA graph."""
    import torch.nn.functional as F

    stream = torch.cuda.current_stream(D.dev)
    xs = x0.reshape(B, 1, H).clone()
    L = len(layers)

    def dense_step():
        xx, r = xs, xs
        for l in layers:
            y = F.linear(F.silu(F.linear(xx, l.wg)) * F.linear(xx, l.wu), l.wdt.t())
            r = r + y
            xx = (r.float() * torch.rsqrt(r.float().pow(2).mean(-1, keepdim=True) + 1e-6)).to(dtype)
        return xx

    g = torch.cuda.CUDAGraph()
    sside = torch.cuda.Stream(D.dev)
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
    ms = statistics.median(event_time_ms(g.replay, max(5, args.steps // 4), stream) for _ in range(3))
    del g
    return ms * 1e3 / L


def decoder_block(family, prompt_len, gen, batches, args, D: Dist, eager=True):
    """Configs 3 / 4: the full decoder (random init, fp16, 32 layers), greedy decode after a
    uniform-random prompt, tokens 2..N timed with CUDA events on the device; CATS MLPs against the
    same decoder with dense MLPs, both replayed from CUDA graphs (and eager at batch 1)."""
    from cats_b200 import decoder as DEC

    t_build = time.perf_counter()
    model = DEC.build_random_model(family, torch.float16, D.dev, seed=args.seed)
    thr = DEC.calibrate(model, 0.5, n_prompts=4, prompt_len=128, seed=args.seed + 1)
    build_s = time.perf_counter() - t_build
    cfg = model.config
    g = torch.Generator(device="cpu")
    g.manual_seed(args.seed + 2)
    out = {"workload": f"{family} decoder, random init N(0, 0.02^2), fp16: {cfg.num_hidden_layers} "
                       f"layers, hidden {cfg.hidden_size}, intermediate {cfg.intermediate_size}, "
                       f"{cfg.num_attention_heads} query / {cfg.num_key_value_heads} KV heads, vocab "
                       f"{cfg.vocab_size}; prompt {prompt_len} uniform-random ids, {gen} greedy tokens; "
                       "CATS at 50 % per-layer thresholds from seeded calibration prompts "
                       "(activate_stats -> device histograms -> set_sparse_threshold)",
           "thresholds_min_max": [min(thr), max(thr)], "build_and_calibrate_s": build_s,
           "timing": "tokens 2..N, CUDA events on the device (time_util_nofile.py:2902-2994)",
           "batches": {}}
    for B in batches:
        ids = torch.randint(0, cfg.vocab_size, (B, prompt_len), generator=g).to(D.dev)
        res = {}
        for mode in ("cats", "dense"):
            dec = DEC.CatsDecoder(model, B, prompt_len + gen + 8, mlp=mode, thresholds=thr)
            dec.prefill(ids)
            _, tps, _ = dec.decode(gen, use_graph=True)
            res[mode] = {"tokens_per_s_graph": tps, "ms_per_token_graph": B * 1e3 / tps}
            if eager and B == 1:
                dec.prefill(ids)
                _, tps_e, _ = dec.decode(min(gen, 128), use_graph=False)
                res[mode]["tokens_per_s_eager"] = tps_e
            if mode == "cats":
                torch.cuda.synchronize()
                res[mode]["device_status"] = dec.ws.counters()[1]
                res[mode]["mlp_launches_per_token"] = dec.mlp_launches_per_step
            del dec
            torch.cuda.empty_cache()
        res["speedup_of_cats_graph"] = res["cats"]["tokens_per_s_graph"] / res["dense"]["tokens_per_s_graph"]
        out["batches"][str(B)] = res
    # the MLP's share of a decode step: the same 32 CATS MLPs alone (cats_mlp per layer, graph)
    del model
    torch.cuda.empty_cache()
    return out


def module_overhead_block(H, I, dtype, D: Dist):
    """Host cost of ``CatsSparseSiluMLP.forward`` per decode call (what HF ``generate`` pays 32
    times per token): wall time per call of a long unsynchronised loop against the kernel's
    device time per call in the same loop."""
    from cats_b200 import sparse_silu as S

    m = S.LlamaSparseSiluMLP({"hidden_size": H, "intermediate_size": I}).to(D.dev, dtype)
    with torch.no_grad():
        for lin in (m.gate_proj, m.up_proj, m.down_proj):
            lin.weight.normal_(0, 0.02)
    m.is_profile, m.sp_method, m.dead_threshold = True, 1, torch.tensor(0.26)
    x = torch.randn(1, 1, H, device=D.dev).to(dtype)
    stream = torch.cuda.current_stream(D.dev)
    with torch.no_grad():
        for _ in range(20):
            m(x)
        torch.cuda.synchronize()
        n = 300
        # host cost: calls issued while the GPU is still busy with earlier ones never wait for it
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n):
            m(x)
        host_us = (time.perf_counter() - t0) / n * 1e6
        e1.record(stream)
        e1.synchronize()
        dev_us = e0.elapsed_time(e1) * 1e3 / n
    del m
    return {"host_us_per_call": host_us, "device_us_per_call": dev_us,
            "what": "CatsSparseSiluMLP.forward, decode, one layer's weights (L2-resident: the "
                    "device time here is not a bandwidth figure), 300 calls without synchronising"}


def run_gpu_arm(args):
    import torch.distributed as dist

    from cats_b200 import _lib, ops, synth

    D = Dist()
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py --impl cats needs a CUDA device (no CPU fallback)")
    torch.cuda.set_device(D.dev)
    if D.world > 1:
        dist.init_process_group("nccl", device_id=D.dev)
    H, I, dtype, L, s = workload_config(args)
    B = args.batch
    esize = torch.empty((), dtype=dtype).element_size()
    stream = torch.cuda.current_stream(D.dev)
    peak, peak_src = hbm_peak()

    # ---- headline: device-resident timing of the stack ---------------------------------------
    head, stack, layers, x0 = measure_stack(args.workload, H, I, dtype, L, s, B, args, D,
                                            regions=args.regions, sample_clocks=True,
                                            parity_layers=min(3, L) if not args.no_parity else 0)
    ms_step, us_layer = head["ms_per_step"], head["us_per_layer"]
    dense_path = D.world == 1 and stack.dense
    stack_launches = stack.launches_per_step
    I_local = head["intermediate_local"]
    persistent = head["kernel"] == "k_cats_mega"

    # ---- end to end through the host-buffer entry point ------------------------------------
    if D.world == 1:
        stack.x_host.copy_(x0.cpu())
        e2e_step = stack.decode_step
        h2d, d2h = stack.h2d_bytes, stack.d2h_bytes
        api = "CatsMLPStack.decode_step (pinned host in/out, cats_mlp_stack C call)"
    else:
        x_host = x0.cpu().pin_memory()
        out_host = torch.empty_like(x_host).pin_memory()

        def e2e_step():
            stack.set_input(x_host)
            stack.run_device()
            out_host.copy_(stack.x, non_blocking=True)
            stream.synchronize()
        h2d = d2h = x_host.numel() * x_host.element_size()
        api = ("FusedTPStack (pinned host in/out, one cats_tp_mlp_stack C call per rank)"
               if persistent else "TPStack (CUDA graph of kernels + NCCL all-reduce)")
    for _ in range(3):
        e2e_step()
    e2e_samples = timed_regions(e2e_step, args.steps, max(3, args.regions // 2), D, stream)
    ms_e2e = statistics.median(e2e_samples)

    # ---- roofline of the kernel that ran in the timed region ------------------------------------
    n_act = head["n_active_mean_per_rank"]
    bytes_layer = head["bytes_per_layer_per_rank"]
    bytes_gate = esize * I_local * H + esize * B * H
    bytes_updown = 2 * esize * n_act * H + 2 * esize * B * H
    ws = stack.ws
    xin = x0.reshape(B, 1, H).clone()
    out = torch.empty_like(xin)
    staged = None
    if B <= 4 and not dense_path:
        reps = max(1, min(10, 320 // L))
        gate_us = graph_launch_us(lambda i: ops.gate(xin, layers[i].wg, layers[i].threshold, ws=ws),
                                  L, reps, stream)
        ops.gate(xin, layers[0].wg, layers[0].threshold, ws=ws)
        updown_us = graph_launch_us(lambda i: ops.updown(xin, layers[i].wu, layers[i].wdt, ws, out=out),
                                    L, reps, stream)
        staged = {
            "k_gate_tma": {"us": gate_us[0], "bytes": bytes_gate, "GBps": bytes_gate / gate_us[0] / 1e3},
            "k_updown_tma": {"us": updown_us[0], "bytes": bytes_updown,
                             "GBps": bytes_updown / updown_us[0] / 1e3},
        }
    if D.world == 1 and stack.dense:
        streamed = head["bytes_streamed_per_layer"]
        kname, launch_us, launch_bytes = "k_dense_stack", ms_step * 1e3, streamed * L
    elif persistent:
        kname, launch_us, launch_bytes = "k_cats_mega", ms_step * 1e3, bytes_layer * L
    elif staged:
        kname = max(staged, key=lambda k: staged[k]["us"])
        launch_us, launch_bytes = staged[kname]["us"], staged[kname]["bytes"]
    else:
        kname, launch_us, launch_bytes = "k_gate + k_updown (per layer)", us_layer, bytes_layer
    achieved = launch_bytes / launch_us / 1e3
    traffic = None
    if persistent and (args.workload, s, B) in NCU_TRAFFIC_RATIO:
        # measured dram bytes / algorithmic bytes of the captured launch, applied to this launch's
        # algorithmic bytes (both grow in proportion to the rows a rank streams)
        traffic = NCU_TRAFFIC_RATIO[(args.workload, s, B)] * launch_bytes
    roofline = {
        "bound": "hbm", "kernel": kname, "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak, "peak_source": peak_src, "traffic": traffic,
        "bytes_per_launch": launch_bytes, "launch_us": launch_us,
        "units_per_launch": f"{L} layers" if (persistent or dense_path) else "1 layer stage",
        "frac_of_8TBps_nominal": achieved / 8000.0,
        "layer": {"bytes": bytes_layer, "us": us_layer, "GBps": bytes_layer / us_layer / 1e3,
                  "frac": bytes_layer / us_layer / 1e3 / peak,
                  "frac_of_8TBps": bytes_layer / us_layer / 1e3 / 8000.0},
        "staged_kernels": staged, "n_active_mean": n_act, "intermediate_local": I_local,
    }

    extra = {}
    if D.world == 1 and not args.no_dense:
        # ---- one layer per launch: what a decoder sees, and the reference's protocol ------------
        if B <= 4 and not dense_path:
            extra["single_layer"] = single_layer_block(layers, x0, B, H, I, dtype, ws, stream, n_act,
                                                       esize, peak)
        # ---- statistics kernel beside the path (threshold calibration): HBM-bound stream --------
        nval = 160 * 1000 * 1000                       # 320 MB of fp16 activations: larger than L2
        vals = torch.nn.functional.silu(torch.randn(nval // 8, device=D.dev) * 1.28).to(dtype).repeat(8)
        edges = torch.cat([torch.tensor([-torch.inf]), torch.linspace(-1, 1, 998),
                           torch.tensor([torch.inf])]).to(D.dev)
        hcounts = torch.zeros(999, dtype=torch.int64, device=D.dev)
        for _ in range(2):
            ops.histogram(vals, edges, hcounts, take_abs=True)
        h_us = per_launch_us(lambda i: ops.histogram(vals, edges, hcounts, take_abs=True), 1, 5, stream)
        hb = vals.numel() * vals.element_size()
        roofline["stats_kernels"] = {"k_histogram": {
            "us": h_us[1], "bytes": hb, "GBps": hb / h_us[1] / 1e3, "frac": hb / h_us[1] / 1e3 / peak,
            "bound": "instruction issue (about 20 instructions per value), not HBM",
            "what": f"|post-activation| histogram of {vals.numel()} {dtype} values "
                    "(SiLU of N(0, 1.28^2)), the reference's 999 bins"}}
        del vals
        # ---- dense cuBLAS MLP of the same shape (context) --------------------------------------
        d_us = dense_stack_us(layers, x0, B, H, dtype, args, D)
        extra["dense_cublas"] = {
            "us_per_layer": d_us, "tokens_per_s": 1e6 / (d_us * L),
            "what": "torch F.linear x3 + SiLU*mul + residual/RMS-norm per layer, CUDA graph",
            "speedup_of_cats": d_us / us_layer}
        extra["module_call"] = module_overhead_block(H, I, dtype, D)

    if D.world > 1 and persistent:
        stack.close()
    del stack, layers
    torch.cuda.empty_cache()

    # ---- the other configurations ---------------------------------------------------------------
    if D.world == 1 and not args.no_sweep:
        extra["sweep"] = sweep_block(args, D)
    if not args.no_config5:
        H5, I5 = synth.SHAPES["llama70b"]
        sub = argparse.Namespace(**vars(args))
        sub.steps, sub.warmup = max(5, min(args.steps, 20)), 3
        c5, st5, l5, _ = measure_stack("llama70b", H5, I5, torch.bfloat16, args.config5_layers, 0.7, 1,
                                       sub, D, regions=5,
                                       parity_layers=2 if not args.no_parity else 0)
        c5["note"] = ("config 5: the 70B-shaped stack, the same layer count at every number of "
                      "GPUs, sharded over the intermediate dimension")
        if D.world > 1 and c5["kernel"] == "k_cats_mega":
            st5.close()
        del st5, l5
        torch.cuda.empty_cache()
        extra["config5"] = c5
    if D.world == 1 and not args.no_decoder:
        extra["decoder"] = {
            "config3": decoder_block("llama", 128, 512, [1], args, D),
            "config4": decoder_block("mistral", 512, 1024, [1, 4, 8], args, D, eager=False),
        }

    def leave():
        """Multi-rank exit: a last barrier, then leave without tearing NCCL down — destroying the
        process group while a captured CUDA graph still references its collectives can block."""
        if D.world > 1:
            torch.cuda.synchronize()
            dist.barrier()
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)

    if D.rank != 0:
        leave()
        return

    cpu = None
    if D.world == 1 and not args.no_cpu_baseline:
        res = time_cpu(H, I, L, s, B, args.seed, args.cpu_sample_layers, seconds=args.cpu_seconds)
        cpu = cpu_baseline_block(res, L, H, I, B)

    launches = stack_launches if dense_path else 1 if persistent else 2 * L
    line = {
        "metric": METRIC, "value": B * 1e3 / ms_step, "unit": UNIT, "n_gpus": D.world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step,
        "ms_per_step_samples": head["ms_per_step_samples"],
        "timed_regions": {"count": len(head["ms_per_step_samples"]), "steps_each": args.steps,
                          "statistic": "median of the regions' per-step times (each the max over ranks)",
                          **spread(head["ms_per_step_samples"])},
        "us_per_layer": us_layer, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": {torch.float16: "f16", torch.bfloat16: "bf16",
                                       torch.float32: "f32"}[dtype] + " storage, f32 accumulate",
        "data": "synthetic", "config": config_block(args, H, I, dtype, L, s, D.world),
        "e2e": {"value": B * 1e3 / ms_e2e, "unit": UNIT, "ms_per_step": ms_e2e,
                "ms_per_step_samples": e2e_samples,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "api": api},
        "gpu_launches": args.steps * len(head["ms_per_step_samples"]) * launches,
        "gpu_launches_per_step": launches,
        "roofline": roofline, "clocks": head["clocks"], "cpu_baseline": cpu,
    }
    if "parity" in head:
        line["parity"] = head["parity"]
    if D.world > 1:
        line["tp"] = {"mode": head["mode"],
                      "nccl_allreduce_variant": head.get("nccl_allreduce_variant")}
    line.update(extra)
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
