"""Weight packing for the CATS decode path: one pass from a Hugging Face ``state_dict`` to the
layout the kernels read, an on-disk format for it, and a loader that reads only a rank's rows.

The kernels want, per layer, three row-major ``(I, H)`` matrices: ``gate_proj.weight``,
``up_proj.weight`` and the *transpose* of ``down_proj.weight`` (``WdT``), so that one active
neuron is one contiguous row in each.  The reference keeps ``down_proj.weight (H, I)`` and, for
its Triton path, a second transposed copy made by the benchmark script
(experiments/bench_sparse_inference_llama.py:76, ``mlp.wdown_t``); its weights are the shared
``nn.Linear`` modules of the original model (experiments/models/sparse_silu/ugly_utils.py:119-131).
Packing once up front avoids holding both copies of Wd, guarantees 16-byte aligned rows and gives
tensor-parallel ranks their row slices without materialising the full matrices.

File format (little endian):
    8 bytes   magic  b"CATSPK01"
    8 bytes   header length n (uint64)
    n bytes   JSON header: {"dtype", "hidden", "intermediate", "layers", "thresholds": [...],
              "align": 256, "offsets": [[wg, wu, wdt] per layer], "meta": {...}}
    padding to a multiple of 256, then the matrices, each ``I * H`` elements row-major, each
    starting on a 256-byte boundary (offsets are absolute file positions).
bf16 is stored as its raw 16-bit patterns.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .synth import Layer
from .tp import shard_bounds

MAGIC = b"CATSPK01"
ALIGN = 256
_DT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
_NP = {"float32": np.float32, "float16": np.float16, "bfloat16": np.uint16}
HF_NAMES = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")


def _transpose(w: torch.Tensor) -> torch.Tensor:
    """(H, I) -> contiguous (I, H); on a GPU through the library's transpose kernel."""
    if w.is_cuda:
        from . import ops

        return ops.transpose(w.contiguous())
    return w.t().contiguous()


def pack_layer(gate_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor, threshold: float = 0.0,
               rank: int = 0, world: int = 1) -> Layer:
    """One layer in kernel layout from the three ``nn.Linear`` weights: gate/up ``(I, H)``,
    down ``(H, I)``.  ``world > 1`` keeps only ``rank``'s rows (``tp.shard_bounds``)."""
    I, H = gate_w.shape
    if tuple(up_w.shape) != (I, H) or tuple(down_w.shape) != (H, I):
        raise RuntimeError("cats_b200.pack: need gate/up (I, H) and down (H, I)")
    lo, hi = shard_bounds(I, rank, world) if world > 1 else (0, I)
    wdt = _transpose(down_w[:, lo:hi]) if world > 1 else _transpose(down_w)
    return Layer(gate_w[lo:hi].contiguous(), up_w[lo:hi].contiguous(), wdt, float(threshold))


def pack_state_dict(state_dict: Dict[str, torch.Tensor], num_layers: Optional[int] = None,
                    prefix: str = "model.layers.{i}.mlp.", thresholds: Optional[Sequence[float]] = None,
                    device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None,
                    rank: int = 0, world: int = 1) -> List[Layer]:
    """All MLP layers of a Llama / Mistral ``state_dict`` (names ``model.layers.N.mlp.
    {gate,up,down}_proj.weight``) in kernel layout, one layer at a time."""
    if num_layers is None:
        num_layers = 0
        while prefix.format(i=num_layers) + HF_NAMES[0] in state_dict:
            num_layers += 1
    if num_layers == 0:
        raise RuntimeError(f"cats_b200.pack: no '{prefix.format(i=0)}{HF_NAMES[0]}' in the state dict")
    layers = []
    for i in range(num_layers):
        ws = []
        for name in HF_NAMES:
            w = state_dict[prefix.format(i=i) + name]
            if device is not None or dtype is not None:
                w = w.to(device=device, dtype=dtype)
            ws.append(w)
        t = float(thresholds[i]) if thresholds is not None else 0.0
        layers.append(pack_layer(ws[0], ws[1], ws[2], t, rank, world))
    return layers


def _raw(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def save_packed(path: str, layers: Sequence[Layer], meta: Optional[dict] = None) -> None:
    """Write unsharded packed layers (``Layer.wg/wu/wdt`` all ``(I, H)``) to ``path``."""
    I, H = layers[0].wg.shape
    dtype = str(layers[0].wg.dtype).replace("torch.", "")
    if dtype not in _DT:
        raise RuntimeError(f"cats_b200.pack: unsupported dtype {dtype}")
    esize = layers[0].wg.element_size()
    mat = (I * H * esize + ALIGN - 1) // ALIGN * ALIGN

    def header(offsets):
        return json.dumps({"dtype": dtype, "hidden": H, "intermediate": I, "layers": len(layers),
                           "thresholds": [float(l.threshold) for l in layers], "align": ALIGN,
                           "offsets": offsets, "meta": meta or {}}).encode()

    # the header's length depends on the offsets' digits: settle it with a second pass
    offsets = [[0, 0, 0] for _ in layers]
    for _ in range(3):
        n = len(header(offsets))
        data0 = (16 + n + ALIGN - 1) // ALIGN * ALIGN
        new = [[data0 + (3 * i + j) * mat for j in range(3)] for i in range(len(layers))]
        if new == offsets:
            break
        offsets = new
    hdr = header(offsets)
    data0 = offsets[0][0]
    if 16 + len(hdr) > data0:
        raise RuntimeError("cats_b200.pack: header did not settle")
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<Q", len(hdr)))
        f.write(hdr)
        f.write(b"\0" * (data0 - 16 - len(hdr)))
        for l in layers:
            for w in (l.wg, l.wu, l.wdt):
                if tuple(w.shape) != (I, H):
                    raise RuntimeError("cats_b200.pack: every matrix must be (I, H)")
                raw = _raw(w)
                f.write(raw.tobytes())
                f.write(b"\0" * (mat - raw.nbytes))
    os.replace(tmp, path)


def read_header(path: str) -> dict:
    with open(path, "rb") as f:
        if f.read(8) != MAGIC:
            raise RuntimeError(f"cats_b200.pack: {path} is not a packed CATS weight file")
        (n,) = struct.unpack("<Q", f.read(8))
        return json.loads(f.read(n).decode())


def load_packed(path: str, device: Optional[torch.device] = None, rank: int = 0, world: int = 1,
                layers: Optional[Sequence[int]] = None) -> List[Layer]:
    """Read packed layers; with ``world > 1`` only ``rank``'s rows of every matrix are read from
    the file (contiguous byte ranges of the memory map)."""
    h = read_header(path)
    H, I, dtype = h["hidden"], h["intermediate"], h["dtype"]
    lo, hi = shard_bounds(I, rank, world) if world > 1 else (0, I)
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    esize = np.dtype(_NP[dtype]).itemsize
    out = []
    for i in (range(h["layers"]) if layers is None else layers):
        ws = []
        for off in h["offsets"][i]:
            a = mm[off + lo * H * esize: off + hi * H * esize].view(_NP[dtype]).reshape(hi - lo, H)
            a = np.array(a)      # a private, writable copy of the mapped bytes
            if dtype == "bfloat16":
                t = torch.from_numpy(a.view(np.int16)).view(torch.bfloat16)
            else:
                t = torch.from_numpy(a)
            ws.append(t.to(device) if device is not None else t)
        out.append(Layer(ws[0], ws[1], ws[2], float(h["thresholds"][i])))
    return out
