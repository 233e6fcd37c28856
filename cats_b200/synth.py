"""Seeded synthetic CATS workloads: weights, decode inputs and calibrated thresholds.

The reference benchmarks on pretrained Llama-2 / Mistral checkpoints with RefinedWeb prompts and
thresholds from activation histograms (experiments/bench_sparse_inference_llama.py:51-77).  None
of that data is available offline, so benches and tests use stand-ins with the real models'
shapes: weights ~ N(0, 0.02^2), decode input x ~ N(0, 1) scaled to unit RMS, and a threshold that
is the requested quantile of |SiLU(Wg x)| pooled over 256 calibration vectors drawn from the same
distribution.  Everything is a pure function of the seed.

This module only prepares data (torch RNG, one matmul for the calibration); it is not part of
the measured path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

# (hidden, intermediate) of the shapes the reference evaluates
SHAPES = {
    "llama7b": (4096, 11008),
    "mistral7b": (4096, 14336),
    "llama70b": (8192, 28672),
}

WEIGHT_STD = 0.02
N_CALIB = 256


@dataclass
class Layer:
    wg: torch.Tensor   # (I, H) gate_proj.weight
    wu: torch.Tensor   # (I, H) up_proj.weight
    wdt: torch.Tensor  # (I, H) down_proj.weight transposed (intermediate-major)
    threshold: float

    @property
    def wd(self) -> torch.Tensor:
        """down_proj.weight in nn.Linear layout (H, I) as a strided view (no copy)."""
        return self.wdt.t()

    def wd_contiguous(self) -> torch.Tensor:
        """down_proj.weight (H, I) as a contiguous tensor (made once, kept): what nn.Linear holds
        and what the dense batched path streams."""
        w = self.__dict__.get("_wd_hi")
        if w is None:
            w = self.wdt.t().contiguous()
            self.__dict__["_wd_hi"] = w
        return w


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def unit_rms(x: torch.Tensor) -> torch.Tensor:
    xf = x.float()
    return (xf / xf.pow(2).mean(-1, keepdim=True).sqrt()).to(x.dtype)


def make_x(B: int, H: int, dtype, device, seed: int) -> torch.Tensor:
    """Decode input (B, 1, H): N(0,1) scaled to unit RMS, rounded to ``dtype``."""
    x = torch.randn((B, 1, H), generator=_gen(device, seed), device=device, dtype=torch.float32)
    return unit_rms(x).to(dtype)


def make_weight(rows: int, cols: int, dtype, device, seed: int, std: float = WEIGHT_STD):
    w = torch.empty((rows, cols), device=device, dtype=dtype)
    # normal_ in the target dtype avoids a transient fp32 copy of multi-GB matrices
    w.normal_(0.0, std, generator=_gen(device, seed))
    return w


def calibrate_threshold(wg: torch.Tensor, sparsity: float, seed: int, n_calib: int = N_CALIB,
                        x_calib: Optional[torch.Tensor] = None) -> float:
    """Quantile ``sparsity`` of |SiLU(Wg x)| pooled over the calibration vectors (fp32)."""
    I, H = wg.shape
    if x_calib is None:
        x_calib = make_x(n_calib, H, wg.dtype, wg.device, seed).reshape(n_calib, H)
    act = torch.nn.functional.silu(x_calib.float() @ wg.float().t()).abs().flatten()
    k = int(sparsity * act.numel())
    if k <= 0:
        return -1.0
    return float(torch.kthvalue(act, k).values)


def make_layer(H: int, I: int, dtype, device, seed: int, sparsity: float = 0.5,
               std: float = WEIGHT_STD) -> Layer:
    wg = make_weight(I, H, dtype, device, seed * 10 + 1, std)
    wu = make_weight(I, H, dtype, device, seed * 10 + 2, std)
    wdt = make_weight(I, H, dtype, device, seed * 10 + 3, std)
    thr = calibrate_threshold(wg, sparsity, seed * 10 + 4)
    return Layer(wg, wu, wdt, thr)


def make_stack(L: int, H: int, I: int, dtype, device, seed: int, sparsity: float = 0.5) -> List[Layer]:
    """L independent layers.  Every layer sees a unit-RMS input (the stack re-normalises between
    layers), so each threshold is calibrated on the same input distribution."""
    return [make_layer(H, I, dtype, device, seed * 1000 + l, sparsity) for l in range(L)]
