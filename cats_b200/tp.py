"""Tensor-parallel CATS MLP: shard the intermediate dimension, one all-reduce per layer.

The MLP output is a sum over intermediate neurons and the threshold test is per neuron, so rank r
of k can own rows [r*I/k, (r+1)*I/k) of Wg, Wu and WdT end to end: it thresholds its own slice
with the *same* threshold, runs stages 1-3 on it and contributes a partial [B, H] output.  The
partials are summed with one all-reduce per layer (NCCL over NVLink when the process group is
NCCL), after which every rank applies the residual add + RMS norm itself (``cats_tail``), so the
next layer's input is replicated again.  The reference has no tensor parallelism (its only
multi-GPU inference mode is HF ``device_map="auto"`` layer placement,
experiments/bench_sparse_inference_llama.py:36); masks per slice are identical to the unsharded
run because nothing crosses ranks before the sum.

``shard_rows`` / ``shard_layer`` are pure tensor slicing and run anywhere; ``TPStack`` drives the
CUDA kernels and a torch.distributed process group.  ``local_mlp`` can be replaced (the CPU tests
plug in a reference implementation to check the sharding algebra under gloo).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .synth import Layer


def shard_bounds(I: int, rank: int, world: int, multiple: int = 32) -> Tuple[int, int]:
    """Row range of ``rank``: contiguous, ascending, boundaries rounded to ``multiple`` rows."""
    if world < 1 or not (0 <= rank < world):
        raise RuntimeError(f"cats_b200.tp: bad rank {rank} of {world}")
    units = (I + multiple - 1) // multiple
    lo = (units * rank // world) * multiple
    hi = (units * (rank + 1) // world) * multiple
    return min(lo, I), min(hi, I)


def shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    lo, hi = shard_bounds(w.shape[0], rank, world)
    return w[lo:hi].contiguous()


def shard_layer(layer: Layer, rank: int, world: int) -> Layer:
    """This rank's slice of a layer; the threshold is global and stays as it is."""
    return Layer(shard_rows(layer.wg, rank, world), shard_rows(layer.wu, rank, world),
                 shard_rows(layer.wdt, rank, world), layer.threshold)


def _cuda_local_mlp(x, layer: Layer, out, ws=None):
    from . import ops

    return ops.mlp(x, layer.wg, layer.wu, layer.wdt, layer.threshold, out=out, ws=ws)


def _cuda_tail(y, resid, x_next, eps):
    from . import ops

    ops.tail(y, resid, x_next, None, eps)


class TPStack:
    """Decode loop of L sharded CATS MLP layers.  Every rank holds ``layers`` already sharded."""

    def __init__(self, layers: Sequence[Layer], batch: int = 1, eps: float = 1e-6,
                 group: Optional[dist.ProcessGroup] = None,
                 local_mlp: Callable = _cuda_local_mlp, tail: Callable = _cuda_tail):
        self.layers: List[Layer] = list(layers)
        self.L = len(self.layers)
        self.H = self.layers[0].wg.shape[1]
        self.dtype, self.device = self.layers[0].wg.dtype, self.layers[0].wg.device
        self.B, self.eps, self.group = batch, eps, group
        self.local_mlp, self.tail = local_mlp, tail
        z = lambda: torch.zeros((batch, self.H), dtype=self.dtype, device=self.device)
        self.x, self.x_tmp, self.resid, self.partial = z(), z(), z(), z()
        self.graph = None
        self.ws = None
        if local_mlp is _cuda_local_mlp:
            from . import ops

            # own workspace: nothing may be allocated while a CUDA graph is being captured
            self.ws = ops.Workspace(self.device, self.H, max(l.wg.shape[0] for l in self.layers))
        self.launches_per_step = 3 * self.L  # stage 1, stages 2+3, tail (+ the all-reduce)

    def set_input(self, x: torch.Tensor) -> None:
        self.x.copy_(x.reshape(self.B, self.H), non_blocking=True)
        self.resid.copy_(self.x, non_blocking=True)

    def _layers_once(self) -> None:
        cur, nxt = self.x, self.x_tmp
        for layer in self.layers:
            self.local_mlp(cur.view(self.B, 1, self.H), layer, self.partial, self.ws)
            if dist.is_initialized() and dist.get_world_size(self.group) > 1:
                dist.all_reduce(self.partial, group=self.group)
            self.tail(self.partial, self.resid, nxt, self.eps)
            cur, nxt = nxt, cur
        if cur is not self.x:
            self.x.copy_(cur)

    def capture(self) -> None:
        """Record one token (all layers, all-reduces included) into a CUDA graph."""
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for _ in range(2):
                self._layers_once()
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._layers_once()
        self.graph = g

    def run_device(self) -> None:
        if self.graph is not None:
            self.graph.replay()
        else:
            self._layers_once()
