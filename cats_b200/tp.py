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

``FusedTPStack`` is the product path: ONE persistent kernel per GPU and token
(``cats_tp_mlp_stack``) whose CTAs push their slice of the layer's partial sums into every peer's
exchange buffer over NVLink, add the ranks' partials of that slice themselves and hand the total
to the other CTAs of their GPU — no collective library call, no kernel boundary between layers.  ``TPStack`` (kernels + one NCCL all-reduce per layer in a CUDA
graph) is kept as the baseline it is measured against.

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


def agree(group: Optional[dist.ProcessGroup] = None, **facts) -> None:
    """Raise on every rank unless all ranks of the group hold the same ``facts`` (hidden size,
    batch, number of layers, dtype ...).  Ranks that disagree would run a different number of
    exchanges, or exchanges of different sizes, and block one another until a time-out; this
    turns that into an immediate error with the differing values named (host side, one
    all_gather of a small object)."""
    if not dist.is_initialized() or dist.get_world_size(group) < 2:
        return
    mine = {k: str(v) for k, v in facts.items()}
    everyone = [None] * dist.get_world_size(group)
    dist.all_gather_object(everyone, mine, group=group)
    bad = [(r, k, o[k], everyone[0][k]) for r, o in enumerate(everyone) for k in mine
           if o.get(k) != everyone[0].get(k)]
    if bad:
        raise RuntimeError("cats_b200.tp: the ranks do not agree on the stack: " + "; ".join(
            f"rank {r} has {k}={v}, rank 0 has {v0}" for r, k, v, v0 in bad))


class PeerLost(RuntimeError):
    """A peer did not report in time (it exited, hangs, or never started)."""


class PeerHeartbeat:
    """Host-side liveness of the ranks of a tensor-parallel group through a key-value store
    (``torch.distributed`` TCPStore / FileStore / HashStore).  Every rank calls ``beat(step)``
    after finishing a step and ``require(step)`` before launching step ``step + 1``: a rank that
    left between steps is then discovered on the host, by name, within ``deadline_s`` - before a
    kernel is launched that would wait for it on the device until its own limit.  No GPU work."""

    def __init__(self, store, rank: int, world: int, deadline_s: float = 5.0,
                 prefix: str = "cats_tp/alive"):
        self.store, self.rank, self.world = store, rank, world
        self.deadline_s, self.prefix = deadline_s, prefix

    def beat(self, step: int) -> None:
        self.store.set(f"{self.prefix}/{self.rank}", str(int(step)))

    def _seen(self, peer: int) -> int:
        key = f"{self.prefix}/{peer}"
        if not self.store.check([key]):
            return -1
        return int(self.store.get(key))

    def require(self, step: int) -> None:
        """Return once every peer has reported ``step`` (or a later one); PeerLost otherwise."""
        import time

        t_end = time.monotonic() + self.deadline_s
        waiting = [p for p in range(self.world) if p != self.rank]
        while waiting:
            waiting = [p for p in waiting if self._seen(p) < step]
            if not waiting:
                return
            if time.monotonic() > t_end:
                raise PeerLost(f"cats_b200.tp: rank(s) {waiting} did not report step {step} "
                               f"within {self.deadline_s} s (rank {self.rank} stops before its "
                               "next launch)")
            time.sleep(0.005)


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
        agree(group, layers=self.L, hidden=self.H, batch=batch, dtype=self.dtype)
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


class ExchangeBuffers:
    """One exchange buffer per rank for ``cats_tp_mlp_stack``: this rank's own (allocated and
    cleared by the library) and the peers' mapped through CUDA IPC handles that travel over the
    process group's host channel (``all_gather_object``)."""

    def __init__(self, H: int, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        import ctypes
        from . import _lib

        L = _lib.lib()
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device
        own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        with torch.cuda.device(device):
            _lib.check(L.cats_tp_exchange_alloc(H, ctypes.byref(own), handle), "exchange alloc")
        self.own = own.value
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.ptrs = []
        for p in range(self.world):
            if p == self.rank:
                self.ptrs.append(self.own)
                continue
            q = ctypes.c_void_p()
            with torch.cuda.device(device):
                _lib.check(L.cats_tp_exchange_open(handles[p], ctypes.byref(q)),
                           f"exchange open (rank {p})")
            self.ptrs.append(q.value)
        self.array = (ctypes.c_void_p * self.world)(*self.ptrs)
        if self.world > 1:
            dist.barrier(group=group)

    def close(self) -> None:
        """Unmap the peers' buffers and free the own one (all ranks, after their last launch)."""
        from . import _lib

        L = _lib.lib()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for p, ptr in enumerate(self.ptrs):
                if p != self.rank and ptr:
                    L.cats_tp_exchange_close(ptr)
            if dist.is_initialized() and self.world > 1:
                dist.barrier()
            if self.own:
                L.cats_tp_exchange_free(self.own)
        self.ptrs, self.own = [], None


class FusedTPStack:
    """Decode loop of L sharded CATS MLP layers as one persistent kernel per GPU and token, the
    ranks exchanging partial sums inside the kernel.  Same interface as ``TPStack``."""

    def __init__(self, layers: Sequence[Layer], batch: int = 1, eps: float = 1e-6,
                 group: Optional[dist.ProcessGroup] = None):
        import ctypes
        from . import _lib, ops

        self.layers: List[Layer] = list(layers)
        self.L = len(self.layers)
        self.H = self.layers[0].wg.shape[1]
        self.I_local = self.layers[0].wg.shape[0]
        if any(l.wg.shape[0] != self.I_local for l in self.layers):
            raise RuntimeError("cats_b200.tp: every layer needs the same number of local rows")
        self.dtype, self.device = self.layers[0].wg.dtype, self.layers[0].wg.device
        self.B, self.eps, self.group = batch, eps, group
        agree(group, layers=self.L, hidden=self.H, batch=batch, dtype=self.dtype)
        z = lambda: torch.zeros((batch, self.H), dtype=self.dtype, device=self.device)
        self.x, self.resid = z(), z()
        self.ws = ops.Workspace(self.device, self.H, self.I_local)
        self.xb = ExchangeBuffers(self.H, self.device, group)
        arr = lambda ts: (ctypes.c_void_p * self.L)(*[t.data_ptr() for t in ts])
        self._wg, self._wu = arr([l.wg for l in self.layers]), arr([l.wu for l in self.layers])
        self._wd = arr([l.wdt for l in self.layers])
        self._thr = (ctypes.c_float * self.L)(*[float(l.threshold) for l in self.layers])
        self._dt = ops.dtype_code(self.dtype)
        self.launches_per_step = 1
        self.failed = False

    def set_input(self, x: torch.Tensor) -> None:
        self.x.copy_(x.reshape(self.B, self.H), non_blocking=True)
        self.resid.copy_(self.x, non_blocking=True)

    def capture(self) -> None:  # one launch per token already
        pass

    def run_device(self) -> None:
        from . import _lib

        if self.failed:
            raise RuntimeError(
                "cats_b200.tp: a wait inside the tensor-parallel kernel ran out earlier; the "
                "workspace and every rank's exchange buffer are invalid - build a new "
                "FusedTPStack on all ranks")
        with torch.cuda.device(self.device):
            st = _lib.lib().cats_tp_mlp_stack(
                self.L, self._wg, self._wu, self._wd, self._thr, self.x.data_ptr(),
                self.resid.data_ptr(), self.ws.ptr, self.ws.nbytes, self.B, self.H, self.I_local,
                self._dt, float(self.eps), self.xb.world, self.xb.rank, self.xb.array,
                torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(st, "cats_tp_mlp_stack")

    def device_status(self) -> int:
        """Sticky device status word (synchronises the stream).  Non-zero: a bounded wait ran
        out (a peer never arrived); this stack refuses further launches."""
        status = self.ws.counters()[1]
        if status != 0:
            self.failed = True
        return status

    def check(self) -> None:
        """Raise if a wait inside the kernel ran out (synchronises the stream)."""
        status = self.device_status()
        if status != 0:
            raise RuntimeError(f"cats_b200.tp: device status {status}: a bounded wait ran out "
                               "inside cats_tp_mlp_stack (peer missing or late); all ranks must "
                               "re-create their exchange buffers and workspaces")

    def close(self) -> None:
        self.xb.close()
