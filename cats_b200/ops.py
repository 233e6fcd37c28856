"""Torch-tensor front end of the C ABI: argument validation, workspace cache, stream plumbing.

Everything here launches on the *current* CUDA stream of the tensors' device and never
synchronises the device.  Tensors are checked (device, dtype, contiguity, shape) and a
``RuntimeError`` is raised on misuse; the reference reinterprets raw ``data_ptr()``s unchecked
(flash_gemv/csrc/cuda/fuse_gemv_cmp_cuda.cu:2332-2336) and exits the process on an unsupported
batch (:2397-2400).

PyTorch is used for device memory and streams only; all arithmetic happens in
``libcats_b200.so``.
"""
from __future__ import annotations

import ctypes
import weakref
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import BF16, F16, F32, MAX_BATCH, OUT_ACC_F32, OUT_STORE

_DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise RuntimeError(f"cats_b200: unsupported dtype {dtype} (float32, float16, bfloat16)")


def _req(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None,
         device: Optional[torch.device] = None) -> None:
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"cats_b200: {name} must be a tensor")
    if not t.is_cuda:
        raise RuntimeError(f"cats_b200: {name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError(f"cats_b200: {name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"cats_b200: {name} has dtype {t.dtype}, expected {dtype}")
    if device is not None and t.device != device:
        raise RuntimeError(f"cats_b200: {name} is on {t.device}, expected {device}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def batch_of(x: torch.Tensor) -> Tuple[int, int]:
    """(B, H) of an activation tensor shaped (B, H), (B, 1, H) or (1, B, H): the reference takes
    B = size(0) * size(1) for 3-D inputs (fuse_gemv_cmp_cuda.cu:2339-2347)."""
    if x.dim() == 3:
        return x.shape[0] * x.shape[1], x.shape[2]
    if x.dim() == 2:
        return x.shape[0], x.shape[1]
    if x.dim() == 1:
        return 1, x.shape[0]
    raise RuntimeError(f"cats_b200: input with {x.dim()} dimensions is not supported")


def _check_batch(B: int) -> None:
    if B < 1 or B > MAX_BATCH:
        raise RuntimeError(f"cats_b200: batch {B} is not supported (1 <= B <= {MAX_BATCH})")


class Workspace:
    """Device scratch shared by the stages of one MLP call (active list, gate values, split-K
    accumulators).  One per (device, stream, H, I); zeroed once, the kernels keep it clean."""

    def __init__(self, device: torch.device, H: int, I: int):
        L = _lib.lib()
        self.H, self.I = H, I
        self.nbytes = int(L.cats_workspace_bytes(MAX_BATCH, H, I))
        self.buf = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)
        self.ptr = self.buf.data_ptr()

    def counters(self) -> Tuple[int, int]:
        """(n_active, device_status) of the latest stage-1 call; synchronises the stream."""
        n, st = ctypes.c_int(0), ctypes.c_int(0)
        with torch.cuda.device(self.buf.device):
            _lib.check(_lib.lib().cats_read_counters(self.ptr, ctypes.byref(n), ctypes.byref(st),
                                                     _stream(self.buf.device)))
        return n.value, st.value


_workspaces = {}


def get_workspace(device: torch.device, H: int, I: int) -> Workspace:
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           _stream(device), H, I)
    ws = _workspaces.get(key)
    if ws is None:
        ws = Workspace(device, H, I)
        _workspaces[key] = ws
    return ws


def clear_workspaces() -> None:
    _workspaces.clear()


class _on:
    """Make ``device`` current for the duration of a launch (cheap when it already is)."""

    def __init__(self, device: torch.device):
        self.idx = device.index
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if self.idx is not None and cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)


# --------------------------------------------------------------------------------------------
# stage wrappers
# --------------------------------------------------------------------------------------------
def gate(x: torch.Tensor, wg: torch.Tensor, threshold: float, gate_dense=None, flag_dense=None,
         ws: Optional[Workspace] = None) -> Workspace:
    """Stage 1 (``cats_gate``).  Returns the workspace that now holds the active list."""
    _req(x, "input")
    dev, dt = x.device, x.dtype
    _req(wg, "gate weight", dt, dev)
    B, H = batch_of(x)
    _check_batch(B)
    if wg.dim() != 2 or wg.shape[1] != H:
        raise RuntimeError(f"cats_b200: gate weight must be (I, {H}), got {tuple(wg.shape)}")
    I = wg.shape[0]
    if gate_dense is not None:
        _req(gate_dense, "output", dt, dev)
        if gate_dense.numel() != B * I:
            raise RuntimeError("cats_b200: output must hold B*I elements")
    if flag_dense is not None:
        _req(flag_dense, "flag", None, dev)
        if flag_dense.dtype not in (torch.bool, torch.uint8) or flag_dense.numel() != B * I:
            raise RuntimeError("cats_b200: flag must be a bool/uint8 tensor with B*I elements")
    ws = ws or get_workspace(dev, H, I)
    with _on(dev):
        _lib.check(_lib.lib().cats_gate(x.data_ptr(), wg.data_ptr(), ws.ptr, ws.nbytes, B, H, I,
                                        dtype_code(dt), float(threshold), _ptr(gate_dense),
                                        _ptr(flag_dense), _stream(dev)), "cats_gate")
    return ws


def compact(values: torch.Tensor, flags: Optional[torch.Tensor], threshold: float, H: int,
            ws: Optional[Workspace] = None) -> Workspace:
    """Active list from dense gate values (``cats_compact``).  values: (..., I) with B*I elements."""
    _req(values, "gate values")
    dev, dt = values.device, values.dtype
    I = values.shape[-1]
    B = values.numel() // I
    _check_batch(B)
    if flags is not None:
        _req(flags, "flag", None, dev)
        if flags.dtype not in (torch.bool, torch.uint8) or flags.numel() != B * I:
            raise RuntimeError("cats_b200: flag must be a bool/uint8 tensor with B*I elements")
    ws = ws or get_workspace(dev, H, I)
    with _on(dev):
        _lib.check(_lib.lib().cats_compact(values.data_ptr(), _ptr(flags), ws.ptr, ws.nbytes, B,
                                           H, I, dtype_code(dt), float(threshold), _stream(dev)),
                   "cats_compact")
    return ws


def up(x: torch.Tensor, wu: torch.Tensor, ws: Workspace, inter_dense=None) -> None:
    """Stage 2 (``cats_up``) over the list held by ``ws``."""
    _req(x, "input")
    dev, dt = x.device, x.dtype
    _req(wu, "up weight", dt, dev)
    B, H = batch_of(x)
    _check_batch(B)
    if wu.dim() != 2 or wu.shape[1] != H or wu.shape[0] != ws.I:
        raise RuntimeError(f"cats_b200: up weight must be ({ws.I}, {H}), got {tuple(wu.shape)}")
    if inter_dense is not None:
        _req(inter_dense, "output", dt, dev)
        if inter_dense.numel() != B * ws.I:
            raise RuntimeError("cats_b200: output must hold B*I elements")
    with _on(dev):
        _lib.check(_lib.lib().cats_up(x.data_ptr(), wu.data_ptr(), ws.ptr, ws.nbytes, B, H, ws.I,
                                      dtype_code(dt), _ptr(inter_dense), _stream(dev)), "cats_up")


def down(wdt: torch.Tensor, ws: Workspace, out: torch.Tensor, B: int,
         accumulate_f32: bool = False) -> None:
    """Stage 3 (``cats_down``): WdT is (I, H); ``out`` holds B*H elements."""
    _req(wdt, "down weight (I, H)")
    dev, dt = wdt.device, wdt.dtype
    _check_batch(B)
    if wdt.dim() != 2 or wdt.shape[0] != ws.I or wdt.shape[1] != ws.H:
        raise RuntimeError(
            f"cats_b200: transposed down weight must be ({ws.I}, {ws.H}), got {tuple(wdt.shape)}")
    _req(out, "output", torch.float32 if accumulate_f32 else dt, dev)
    if out.numel() != B * ws.H:
        raise RuntimeError("cats_b200: output must hold B*H elements")
    with _on(dev):
        _lib.check(_lib.lib().cats_down(wdt.data_ptr(), ws.ptr, ws.nbytes, B, ws.H, ws.I,
                                        dtype_code(dt), out.data_ptr(),
                                        OUT_ACC_F32 if accumulate_f32 else OUT_STORE,
                                        _stream(dev)), "cats_down")


def _check_mlp_weights(x, wg, wu, wdt):
    _req(x, "input")
    dev, dt = x.device, x.dtype
    B, H = batch_of(x)
    _check_batch(B)
    _req(wg, "gate weight", dt, dev)
    _req(wu, "up weight", dt, dev)
    _req(wdt, "down weight (I, H)", dt, dev)
    if wg.dim() != 2 or wg.shape[1] != H:
        raise RuntimeError(f"cats_b200: gate weight must be (I, {H}), got {tuple(wg.shape)}")
    I = wg.shape[0]
    if tuple(wu.shape) != (I, H):
        raise RuntimeError(f"cats_b200: up weight must be ({I}, {H}), got {tuple(wu.shape)}")
    if tuple(wdt.shape) != (I, H):
        raise RuntimeError(
            f"cats_b200: transposed down weight must be ({I}, {H}), got {tuple(wdt.shape)}")
    return dev, dt, B, H, I


def updown(x, wu, wdt, ws: Workspace, out: Optional[torch.Tensor] = None,
           accumulate_f32: bool = False, resid=None, x_next=None, norm_weight=None,
           eps: float = 1e-6) -> torch.Tensor:
    """Stages 2+3 in one launch (``cats_updown``) over the list held by ``ws``."""
    dev, dt, B, H, I = _check_mlp_weights(x, wu, wu, wdt)
    if out is None and resid is None:
        out = torch.empty_like(x)
    for t, name in ((resid, "resid"), (x_next, "x_next")):
        if t is not None:
            _req(t, name, dt, dev)
            if t.numel() != B * H:
                raise RuntimeError(f"cats_b200: {name} must hold B*H elements")
    if out is not None:
        _req(out, "output", torch.float32 if accumulate_f32 else dt, dev)
        if out.numel() != B * H:
            raise RuntimeError("cats_b200: output must hold B*H elements")
    if norm_weight is not None:
        _req(norm_weight, "norm weight", dt, dev)
    with _on(dev):
        _lib.check(_lib.lib().cats_updown(x.data_ptr(), wu.data_ptr(), wdt.data_ptr(), ws.ptr,
                                          ws.nbytes, B, H, I, dtype_code(dt), _ptr(out),
                                          OUT_ACC_F32 if accumulate_f32 else OUT_STORE,
                                          _ptr(resid), _ptr(x_next), _ptr(norm_weight),
                                          float(eps), _stream(dev)), "cats_updown")
    return out


def mlp(x, wg, wu, wdt, threshold: float, out: Optional[torch.Tensor] = None,
        accumulate_f32: bool = False, resid=None, x_next=None, norm_weight=None,
        eps: float = 1e-6, ws: Optional[Workspace] = None) -> torch.Tensor:
    """The whole CATS MLP for decode (``cats_mlp``): x (B,H)/(B,1,H); wg, wu, wdt all (I, H).

    Computes ``Wd @ (mask(SiLU(Wg x)) * (Wu x))`` with mask = ``|.| > threshold`` — the dense
    thresholded MLP of experiments/models/sparse_silu/ugly_utils.py:896-899 — reading only the
    active rows of wu and wdt.  Returns a new tensor shaped like ``x`` unless ``out`` is given.
    """
    dev, dt, B, H, I = _check_mlp_weights(x, wg, wu, wdt)
    if out is None and resid is None:
        out = torch.empty_like(x)
    for t, name in ((resid, "resid"), (x_next, "x_next")):
        if t is not None:
            _req(t, name, dt, dev)
            if t.numel() != B * H:
                raise RuntimeError(f"cats_b200: {name} must hold B*H elements")
    if out is not None:
        _req(out, "output", torch.float32 if accumulate_f32 else dt, dev)
        if out.numel() != B * H:
            raise RuntimeError("cats_b200: output must hold B*H elements")
    if norm_weight is not None:
        _req(norm_weight, "norm weight", dt, dev)
    ws = ws or get_workspace(dev, H, I)
    with _on(dev):
        _lib.check(_lib.lib().cats_mlp(x.data_ptr(), wg.data_ptr(), wu.data_ptr(), wdt.data_ptr(),
                                       ws.ptr, ws.nbytes, B, H, I, dtype_code(dt),
                                       float(threshold), _ptr(out),
                                       OUT_ACC_F32 if accumulate_f32 else OUT_STORE, _ptr(resid),
                                       _ptr(x_next), _ptr(norm_weight), float(eps), _stream(dev)),
                   "cats_mlp")
    return out


# Which path a batch takes when the caller holds down_proj.weight in both layouts.  The sparse
# kernels stream all of Wg plus the union of the tokens' active rows of Wu and WdT, at about 0.55
# of the HBM peak for batches of 2-4 (measured); the dense tensor-core path streams all three
# matrices at about 0.75.  Equal time at a union density of about 0.6; beyond four tokens the
# sparse path has no tensor-core kernel and the dense path always wins.
DENSE_UNION_DENSITY = 0.6


def use_dense(B: int, sparsity: Optional[float] = None, union_density: Optional[float] = None) -> bool:
    """Density-aware switch between the sparse kernels and the dense tensor-core path.
    ``union_density``: expected fraction of neurons active for at least one of the B tokens;
    when unknown it is estimated from the per-token ``sparsity`` (default 0.5) as if the tokens'
    masks were independent, 1 - sparsity**B (the reference tracks the measured quantity as
    ``agg_sparsity``, experiments/models/sparse_silu/ugly_utils.py:594)."""
    if B < 2:
        return False
    if B > 4:
        return True
    if union_density is None:
        s = 0.5 if sparsity is None else min(max(float(sparsity), 0.0), 1.0)
        union_density = 1.0 - s ** B
    return union_density >= DENSE_UNION_DENSITY


def dense_supported(B: int, H: int, I: int, dtype: torch.dtype) -> bool:
    """Whether ``mlp_dense`` can run this shape (16-bit weights, H % 128 == 0, H <= 8192, I % 64 == 0)."""
    if dtype not in (torch.float16, torch.bfloat16):
        return False
    return _lib.lib().cats_dense_supported(B, H, I, dtype_code(dtype)) == 1


def mlp_dense(x, wg, wu, wd, threshold: float, out: Optional[torch.Tensor] = None, resid=None,
              x_next=None, norm_weight=None, eps: float = 1e-6,
              ws: Optional[Workspace] = None) -> torch.Tensor:
    """The CATS MLP for a batch on the tensor cores (``cats_mlp_dense``): every weight row is
    streamed, each token's own mask ``|SiLU(gate)| > threshold`` is applied to its products.
    x (B,H)/(B,1,H)/(1,B,H); wg, wu (I, H); wd (H, I) = down_proj.weight as nn.Linear stores it."""
    _req(x, "input")
    dev, dt = x.device, x.dtype
    B, H = batch_of(x)
    _check_batch(B)
    _req(wg, "gate weight", dt, dev)
    _req(wu, "up weight", dt, dev)
    _req(wd, "down weight (H, I)", dt, dev)
    I = wg.shape[0]
    if tuple(wg.shape) != (I, H) or tuple(wu.shape) != (I, H) or tuple(wd.shape) != (H, I):
        raise RuntimeError(f"cats_b200: expected gate/up ({I}, {H}) and down ({H}, {I}), got "
                           f"{tuple(wg.shape)}, {tuple(wu.shape)}, {tuple(wd.shape)}")
    if out is None and resid is None:
        out = torch.empty_like(x)
    for t, name in ((out, "output"), (resid, "resid"), (x_next, "x_next")):
        if t is not None:
            _req(t, name, dt, dev)
            if t.numel() != B * H:
                raise RuntimeError(f"cats_b200: {name} must hold B*H elements")
    if norm_weight is not None:
        _req(norm_weight, "norm weight", dt, dev)
    ws = ws or get_workspace(dev, H, I)
    with _on(dev):
        _lib.check(_lib.lib().cats_mlp_dense(x.data_ptr(), wg.data_ptr(), wu.data_ptr(), wd.data_ptr(),
                                             ws.ptr, ws.nbytes, B, H, I, dtype_code(dt),
                                             float(threshold), _ptr(out), OUT_STORE, _ptr(resid),
                                             _ptr(x_next), _ptr(norm_weight), float(eps),
                                             _stream(dev)), "cats_mlp_dense")
    return out


def down_dense(inter: torch.Tensor, wd: torch.Tensor, out: Optional[torch.Tensor] = None):
    """Dense down projection over Wd (H, I) (``cats_down_dense``); inter holds B*I elements."""
    _req(inter, "intermediate")
    dev, dt = inter.device, inter.dtype
    _req(wd, "down weight (H, I)", dt, dev)
    H, I = wd.shape
    B = inter.numel() // I
    _check_batch(B)
    if out is None:
        out = torch.empty((B, H), dtype=dt, device=dev)
    _req(out, "output", dt, dev)
    with _on(dev):
        _lib.check(_lib.lib().cats_down_dense(inter.data_ptr(), wd.data_ptr(), B, H, I,
                                              dtype_code(dt), out.data_ptr(), _stream(dev)),
                   "cats_down_dense")
    return out


def tail(y: torch.Tensor, resid: torch.Tensor, x_next: Optional[torch.Tensor] = None,
         norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6) -> None:
    """resid += y; x_next = rmsnorm(resid) (``cats_tail``); all tensors hold B*H elements."""
    _req(y, "y")
    dev, dt = y.device, y.dtype
    B, H = batch_of(y)
    _req(resid, "resid", dt, dev)
    if resid.numel() != B * H:
        raise RuntimeError("cats_b200: resid must hold B*H elements")
    if x_next is not None:
        _req(x_next, "x_next", dt, dev)
    if norm_weight is not None:
        _req(norm_weight, "norm weight", dt, dev)
    with _on(dev):
        _lib.check(_lib.lib().cats_tail(y.data_ptr(), resid.data_ptr(), _ptr(x_next),
                                        _ptr(norm_weight), float(eps), B, H, dtype_code(dt),
                                        _stream(dev)), "cats_tail")


def rope_cache(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor,
               q_out: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor, n_heads: int,
               n_kv_heads: int) -> None:
    """RoPE of one new position's query / key heads and the KV-cache write (``cats_rope_cache``).
    qkv (B, (nh + 2 nkv) hd); cos, sin (max_len, hd); pos: int64 CUDA tensor with one element;
    q_out (B, nh, hd); kc, vc (B, nkv, max_len, hd)."""
    _req(qkv, "qkv")
    dev, dt = qkv.device, qkv.dtype
    for t, name in ((cos, "cos"), (sin, "sin"), (q_out, "q_out"), (kc, "key cache"), (vc, "value cache")):
        _req(t, name, dt, dev)
    if pos.dtype != torch.int64 or pos.device != dev or pos.numel() != 1:
        raise RuntimeError("cats_b200: pos must be a one-element int64 tensor on the same device")
    B, nkv, max_len, hd = kc.shape
    if tuple(vc.shape) != tuple(kc.shape) or nkv != n_kv_heads or qkv.numel() != B * (n_heads + 2 * nkv) * hd \
            or q_out.numel() != B * n_heads * hd or tuple(cos.shape) != (max_len, hd) \
            or tuple(sin.shape) != (max_len, hd):
        raise RuntimeError("cats_b200: rope_cache shapes do not fit together")
    with _on(dev):
        _lib.check(_lib.lib().cats_rope_cache(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                              pos.data_ptr(), q_out.data_ptr(), kc.data_ptr(),
                                              vc.data_ptr(), B, n_heads, nkv, hd, max_len,
                                              dtype_code(dt), _stream(dev)), "cats_rope_cache")


def transpose(src: torch.Tensor) -> torch.Tensor:
    """(R, C) -> new contiguous (C, R) through ``cats_transpose``."""
    _req(src, "matrix")
    if src.dim() != 2:
        raise RuntimeError("cats_b200: transpose expects a 2-D tensor")
    R, C = src.shape
    dst = torch.empty((C, R), dtype=src.dtype, device=src.device)
    with _on(src.device):
        _lib.check(_lib.lib().cats_transpose(src.data_ptr(), dst.data_ptr(), R, C,
                                             dtype_code(src.dtype), _stream(src.device)),
                   "cats_transpose")
    return dst


def histogram(values: torch.Tensor, edges: torch.Tensor, counts: Optional[torch.Tensor] = None,
              take_abs: bool = False) -> torch.Tensor:
    """``counts += torch.histogram(values [abs], bins=edges)`` on the device (``cats_histogram``).

    ``edges``: ascending float32 CUDA tensor (the reference's -inf, linspace(-1, 1, 998), +inf);
    ``counts``: int64 CUDA tensor of len(edges) - 1, created (zero) when omitted.  Replaces the
    host-side torch.histogram calls of collect_stats (ugly_utils.py:514-522)."""
    _req(values, "values")
    dev = values.device
    if edges.dtype != torch.float32 or edges.device != dev or not edges.is_contiguous() or edges.dim() != 1:
        raise RuntimeError("cats_b200: histogram edges must be a contiguous 1-D float32 tensor on the values' device")
    if counts is None:
        counts = torch.zeros(edges.numel() - 1, dtype=torch.int64, device=dev)
    if counts.dtype != torch.int64 or counts.device != dev or not counts.is_contiguous() \
            or counts.numel() != edges.numel() - 1:
        raise RuntimeError("cats_b200: histogram counts must be int64[len(edges) - 1] on the values' device")
    with _on(dev):
        _lib.check(_lib.lib().cats_histogram(values.data_ptr(), values.numel(), dtype_code(values.dtype),
                                             edges.data_ptr(), edges.numel(), counts.data_ptr(),
                                             1 if take_abs else 0, _stream(dev)), "cats_histogram")
    return counts


def histogram_threshold(counts: torch.Tensor, edges: torch.Tensor, sparsity: float) -> torch.Tensor:
    """0-dim float32 CUDA tensor: the bin edge at which the histogram's CDF crosses ``sparsity``
    (``cats_histogram_threshold``; get_threshold, ugly_utils.py:236-245, without leaving the device)."""
    dev = counts.device
    if counts.dtype != torch.int64 or not counts.is_cuda or not counts.is_contiguous():
        raise RuntimeError("cats_b200: histogram counts must be a contiguous int64 CUDA tensor")
    if edges.dtype != torch.float32 or edges.device != dev or edges.numel() != counts.numel() + 1 \
            or not edges.is_contiguous():
        raise RuntimeError("cats_b200: need len(counts) + 1 float32 edges on the same device")
    out = torch.empty((), dtype=torch.float32, device=dev)
    with _on(dev):
        _lib.check(_lib.lib().cats_histogram_threshold(counts.data_ptr(), edges.data_ptr(), edges.numel(),
                                                       float(sparsity), out.data_ptr(), _stream(dev)),
                   "cats_histogram_threshold")
    return out


# Packed WdT per down_proj weight.  An entry belongs to one live tensor object: it is found again
# only by that same object (a weak reference is compared, not the address - the caching allocator
# hands the address of a freed weight to the next tensor of the same shape), it is re-packed when
# the tensor was modified in place (version counter) and it is dropped, together with its
# (I, H) copy on the GPU, when the weight tensor is garbage collected.
_packed = {}


def packed_wdt(wd: torch.Tensor) -> torch.Tensor:
    """WdT (I, H) for a down_proj weight given in nn.Linear layout (H, I); packed on first use."""
    key = id(wd)
    hit = _packed.get(key)
    if hit is not None and hit[0]() is wd and hit[1] == wd._version and hit[2] == wd.data_ptr():
        return hit[3]
    _req(wd, "down weight (H, I)")
    wdt = transpose(wd)
    ref = weakref.ref(wd, lambda _r, k=key: _packed.pop(k, None))
    _packed[key] = (ref, wd._version, wd.data_ptr(), wdt)
    return wdt


def clear_packed() -> None:
    _packed.clear()


def export_list(ws: Workspace, B: int, dtype: torch.dtype, idx_out: torch.Tensor,
                val_out: Optional[torch.Tensor]) -> int:
    """Flatten the active list of the latest stage-1 call into idx_out (int64) / val_out and
    return its length (synchronises the stream, like fuse_gemv_cmp in the reference)."""
    dev = ws.buf.device
    _req(idx_out, "idx", torch.int64, dev)
    if val_out is not None:
        _req(val_out, "output", dtype, dev)
    n, _ = ws.counters()
    if idx_out.numel() < n or (val_out is not None and val_out.numel() < n):
        raise RuntimeError("cats_b200: idx/output are smaller than the active list")
    with _on(dev):
        _lib.check(_lib.lib().cats_export_list(ws.ptr, ws.nbytes, B, ws.H, ws.I,
                                               dtype_code(dtype), idx_out.data_ptr(),
                                               _ptr(val_out), _stream(dev)), "cats_export_list")
    return n
