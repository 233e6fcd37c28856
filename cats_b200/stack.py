"""A stack of CATS MLP layers driven through ``cats_mlp_stack`` (one C call per decoded token).

This is the decode loop of the MLP halves of a decoder: for every layer, the CATS MLP of the
RMS-normalised residual is added back to the residual (the reference's decoder layer does
norm -> mlp -> residual add, experiments/models/sparse_silu/ugly_utils.py:1036-1057).  The
residual add and the next layer's RMS norm are fused into the kernel: where the shape allows,
the whole stack is ONE launch of the persistent cooperative kernel per token
(``launches_per_step``), else a stage-1 and a stage-2/3 launch per layer.

``CatsMLPStack.decode_step`` is the host-buffer entry point: it copies the token's hidden state
from pinned host memory, runs all layers and copies the result back.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from . import _lib, ops
from .synth import Layer


class CatsMLPStack:
    """``dense``: None = decided by ``ops.use_dense(batch, sparsity)``; True / False force the
    dense tensor-core path (``cats_mlp_stack_dense``: one cooperative launch for the stack) or the
    sparse kernels."""

    def __init__(self, layers: Sequence[Layer], batch: int = 1, eps: float = 1e-6,
                 dense: Optional[bool] = None, sparsity: Optional[float] = None):
        if not layers:
            raise RuntimeError("cats_b200: empty layer stack")
        l0 = layers[0]
        self.layers: List[Layer] = list(layers)
        self.L = len(self.layers)
        self.I, self.H = l0.wg.shape
        self.dtype, self.device = l0.wg.dtype, l0.wg.device
        self.B = batch
        self.eps = eps
        for l in self.layers:
            for w in (l.wg, l.wu, l.wdt):
                ops._req(w, "layer weight", self.dtype, self.device)
                if tuple(w.shape) != (self.I, self.H):
                    raise RuntimeError("cats_b200: all layers of a stack must share (I, H)")
        ops._check_batch(batch)
        self.code = ops.dtype_code(self.dtype)
        arr = ctypes.c_void_p * self.L
        self._wg = arr(*[l.wg.data_ptr() for l in self.layers])
        self._wu = arr(*[l.wu.data_ptr() for l in self.layers])
        self._wdt = arr(*[l.wdt.data_ptr() for l in self.layers])
        self._thr = (ctypes.c_float * self.L)(*[float(l.threshold) for l in self.layers])
        self.ws = ops.Workspace(self.device, self.H, self.I)
        self.x = torch.zeros((batch, self.H), dtype=self.dtype, device=self.device)
        self.x_tmp = torch.zeros_like(self.x)
        self.resid = torch.zeros_like(self.x)
        self.x_host = torch.zeros((batch, self.H), dtype=self.dtype).pin_memory()
        self.out_host = torch.zeros((batch, self.H), dtype=self.dtype).pin_memory()
        self.h2d_bytes = self.x_host.numel() * self.x_host.element_size()
        self.d2h_bytes = self.out_host.numel() * self.out_host.element_size()
        persistent = _lib.lib().cats_uses_persistent_kernel(self.L, batch, self.H, self.I, self.code)
        self.launches_per_step = 1 if persistent == 1 else 2 * self.L
        want = ops.use_dense(batch, sparsity) if dense is None else bool(dense)
        self.dense = want and ops.dense_supported(batch, self.H, self.I, self.dtype)
        self.graph = None
        if self.dense:
            self._wd = [l.wd_contiguous() for l in self.layers]
            self._wd_ptrs = arr(*[w.data_ptr() for w in self._wd])
            self.launches_per_step = (self.L + 79) // 80     # one cooperative launch per 80 layers

    def _dense_layers(self) -> None:
        cur, nxt = self.x, self.x_tmp
        for l, wd in zip(self.layers, self._wd):
            ops.mlp_dense(cur, l.wg, l.wu, wd, l.threshold, resid=self.resid, x_next=nxt,
                          eps=self.eps, ws=self.ws)
            cur, nxt = nxt, cur
        if cur is not self.x:
            self.x.copy_(cur)

    def capture(self) -> None:
        """Dense path: record the layers' launches into a CUDA graph (the state is restored)."""
        if not self.dense or self.graph is not None:
            return
        keep = (self.x.clone(), self.resid.clone())
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self._dense_layers()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._dense_layers()
        self.graph = g
        self.x.copy_(keep[0])
        self.resid.copy_(keep[1])

    def run_device(self) -> None:
        """All layers on the state already in ``self.x`` / ``self.resid`` (device resident)."""
        if self.dense:
            with ops._on(self.device):
                _lib.check(_lib.lib().cats_mlp_stack_dense(
                    self.L, self._wg, self._wu, self._wd_ptrs, self._thr, self.x.data_ptr(),
                    self.x_tmp.data_ptr(), self.resid.data_ptr(), self.ws.ptr, self.ws.nbytes,
                    self.B, self.H, self.I, self.code, self.eps, ops._stream(self.device)),
                    "cats_mlp_stack_dense")
            return
        with ops._on(self.device):
            _lib.check(_lib.lib().cats_mlp_stack(
                self.L, self._wg, self._wu, self._wdt, self._thr, self.x.data_ptr(),
                self.x_tmp.data_ptr(), self.resid.data_ptr(), self.ws.ptr, self.ws.nbytes,
                self.B, self.H, self.I, self.code, self.eps, ops._stream(self.device)),
                "cats_mlp_stack")

    def set_input(self, x: torch.Tensor) -> None:
        """Start a token: the residual stream and the first layer's input are both ``x``."""
        self.x.copy_(x.reshape(self.B, self.H), non_blocking=True)
        self.resid.copy_(self.x, non_blocking=True)

    def decode_step(self, x_host: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Host buffers in, host buffers out: H2D copy of the token's hidden state, all layers,
        D2H copy of the normalised residual after the last layer.  Blocks until it is there."""
        src = self.x_host if x_host is None else x_host
        self.set_input(src)
        self.run_device()
        self.out_host.copy_(self.x, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return self.out_host

    def active_counts(self) -> List[int]:
        """Active neurons per layer for the state currently in ``self.x`` (runs the layers one
        by one and reads the counter back; for reporting, not for timing)."""
        counts = []
        x, r = self.x.clone(), self.resid.clone()
        nxt = torch.empty_like(x)
        for l in self.layers:
            ops.mlp(x.reshape(self.B, 1, self.H), l.wg, l.wu, l.wdt, l.threshold, resid=r,
                    x_next=nxt, eps=self.eps, ws=self.ws)
            counts.append(self.ws.counters()[0])
            x, nxt = nxt, x
        return counts
