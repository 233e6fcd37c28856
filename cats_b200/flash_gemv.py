"""The reference's ``flash_gemv`` operator API, backed by the sm_100a kernels.

Every public name of the reference package (flash_gemv/flash_gemv/__init__.py:62-80) exists here
with the same positional arguments, tensor layouts and return convention, so
``import flash_gemv`` (the alias package at the repository root) keeps the reference's callers
working: experiments/models/sparse_silu/ugly_utils.py:880-894 and flash_gemv/test, flash_gemv/bench.

Differences that a caller can observe:
* errors are ``RuntimeError``s (wrong device / dtype / layout / batch); the reference prints and
  calls ``exit(-1)`` (fuse_gemv_cmp_cuda.cu:2096-2097, 2397-2400);
* shapes are generic (the reference hard-codes 4096 x 14336 in several ops,
  flash_gemv/csrc/fuse_gemv_cmp.cpp:12-15, 28-45) and any batch 1..16 works;
* products and sums are fp32 (the reference forms 16-bit products, fuse_gemv_cmp_cuda.cu:1327-1329);
* ``fuse_gemv_cmp`` returns its index list in ascending order (unordered in the reference,
  fuse_gemv_cmp_cuda.cu:81);
* nothing synchronises the device and nothing is allocated per call except the returned tensor
  (the reference does cudaMalloc/cudaFree per call, fuse_gemv_cmp_cuda.cu:2351-2354, 2402-2403);
* there is no Triton: ``*_triton`` and ``*_dejavu`` names run the same CUDA kernels.

Entry points that receive ``down_proj.weight`` in nn.Linear layout (H, I) — ``flag_gemv_gemv`` and
``flag_gemv_gemv_inner*`` — pack it once into the intermediate-major WdT (I, H) that the sparse
down projection needs and cache the packed copy per weight tensor (see ``ops.packed_wdt``).  The
``*_triton`` / ``*_dejavu`` names receive ``Wgate`` as (H, I) and pack it the same way.
"""
from __future__ import annotations

import torch

from . import ops

__all__ = [
    "fuse_gemv_cmp", "fuse_gemv_flag", "fuse_gemv_flag_gemv", "fuse_gemv_flag_gemv_gemv",
    "fuse_gemv_gemv_gemv", "fuse_gemv_flag_batch", "fuse_gemv_flag_local", "fuse_flag_gemv_local",
    "atomic_gemv", "flag_gemv_gemv_atomic", "flag_gemv_gemv", "flag_gemv_gemv_inner",
    "flag_gemv_gemv_inner_fp32", "flag_gemv_gemv_inner_bf16", "flag_gemv_gemv_triton",
    "gemv_gemv_triton", "flag_gemv_gemv_fuse_dejavu", "flag_gemv_gemv_dejavu",
]


def _thr(threshold) -> float:
    return float(threshold)


def _as_flag(flag: torch.Tensor) -> torch.Tensor:
    # bool and uint8 share the one-byte 0/1 representation the kernels read and write
    return flag


# ---- stage-1 ops ------------------------------------------------------------------------------
def fuse_gemv_cmp(input, weight, output, idx, threshold):
    """Compacted (value, index) list of the active neurons; returns their count.
    Reference: flash_gemv/flash_gemv/flash_gemv.py:3-4, fuse_gemv_cmp_cuda.cu:43-88, 1962-1977."""
    ws = ops.gate(input, weight, _thr(threshold))
    B, _ = ops.batch_of(input)
    return ops.export_list(ws, B, input.dtype, idx, output)


def fuse_gemv_flag(input, weight, output, flag, threshold):
    """output[i] = SiLU(weight[i,:] . input) for every neuron, flag[i] = |output[i]| > threshold.
    Reference: flash_gemv.py:6-7, fuse_gemv_cmp_cuda.cu:419-456, 1979-2007."""
    ops.gate(input, weight, _thr(threshold), gate_dense=output, flag_dense=_as_flag(flag))


def fuse_gemv_flag_batch(input, weight, output, flag, threshold):
    """Batched fuse_gemv_flag: output / flag are (1, B, I).
    Reference: flash_gemv.py:18-19, fuse_gemv_cmp_cuda.cu:1246-1287, 2058-2077."""
    ops.gate(input, weight, _thr(threshold), gate_dense=output, flag_dense=_as_flag(flag))


def fuse_gemv_flag_local(input, weight, output, flag, threshold):
    """Stage 1 of the model-facing pipeline (gate value rounded to the input dtype + flag).
    Reference: flash_gemv.py:21-22, fuse_gemv_cmp_cuda.cu:1292-1486, 2083-2117."""
    ops.gate(input, weight, _thr(threshold), gate_dense=output, flag_dense=_as_flag(flag))


# ---- stage-2 / stage-3 ops --------------------------------------------------------------------
def fuse_flag_gemv_local(input, weight, output, flag):
    """In place: ``output`` holds the gate values on entry and gate * (weight[i,:] . input) on
    return, 0 where flag is false.  Reference: flash_gemv.py:24-25, fuse_gemv_cmp_cuda.cu:1507-1722."""
    _, H = ops.batch_of(input)
    ws = ops.compact(output, _as_flag(flag), 0.0, H)
    output.zero_()
    ops.up(input, weight, ws, inter_dense=output)


def atomic_gemv(input, weight, output, flag):
    """output (fp32, pre-zeroed by the caller) += sum over flagged i of input[b,i] * weight[i,:],
    weight = Wd transposed (I, H).  Reference: flash_gemv.py:27-28, fuse_gemv_cmp_cuda.cu:1724-1783."""
    I, H = weight.shape
    B = input.numel() // I
    ws = ops.compact(input, _as_flag(flag), 0.0, H)
    ops.down(weight, ws, output, B, accumulate_f32=True)


# ---- fused pipelines --------------------------------------------------------------------------
def fuse_gemv_flag_gemv(input, wgate, wup, output, flag, threshold):
    """Stages 1+2: output[i] = SiLU(gate_i) * up_i and flag[i] = 1 for active neurons; inactive
    entries of ``output`` are left as the caller initialised them (the reference's convention).
    Reference: flash_gemv.py:9-10, fuse_gemv_cmp_cuda.cu:715-784, 2009-2023."""
    ws = ops.gate(input, wgate, _thr(threshold), flag_dense=_as_flag(flag))
    ops.up(input, wup, ws, inter_dense=output)


def fuse_gemv_flag_gemv_gemv(input, wgate, wup, wdown, output, flag, threshold):
    """All three stages; wdown is (I, H); output is fp32, pre-zeroed, accumulated into.
    Reference: flash_gemv.py:12-13, fuse_gemv_cmp_cuda.cu:786-877, 2025-2038."""
    ws = ops.gate(input, wgate, _thr(threshold), flag_dense=_as_flag(flag))
    ops.updown(input, wup, wdown, ws, out=output, accumulate_f32=True)


def fuse_gemv_gemv_gemv(input, wgate, wup, wdown, output, threshold):
    """As above without the flag output.  Reference: flash_gemv.py:15-16,
    fuse_gemv_cmp_cuda.cu:1152-1244, 2040-2056."""
    ops.mlp(input, wgate, wup, wdown, _thr(threshold), out=output, accumulate_f32=True)


def flag_gemv_gemv_atomic(input, wgate, wup, wdown, output, threshold):
    """Three-kernel pipeline with the sparse down projection; wdown (I, H); output fp32
    pre-zeroed.  Reference: flash_gemv.py:30-31, fuse_gemv_cmp_cuda.cu:2196-2253."""
    ops.mlp(input, wgate, wup, wdown, _thr(threshold), out=output, accumulate_f32=True)


def _dense_batch(input, wgate, wdown) -> bool:
    """Batches take the dense tensor-core path where it is supported: these entry points receive
    down_proj.weight as (H, I), which is what that path streams (and, like the reference's
    stage 3 for these names, it reads all of it)."""
    B, H = ops.batch_of(input)
    return (ops.use_dense(B) and wdown.is_contiguous()
            and ops.dense_supported(B, H, wgate.shape[0], input.dtype))


def flag_gemv_gemv(input, wgate, wup, wdown, output, threshold):
    """Three-kernel pipeline writing ``output`` (same dtype as input); wdown is (H, I).
    Reference: flash_gemv.py:33-34, fuse_gemv_cmp_cuda.cu:2255-2328."""
    if _dense_batch(input, wgate, wdown):
        ops.mlp_dense(input, wgate, wup, wdown, _thr(threshold), out=output)
        return
    ops.mlp(input, wgate, wup, ops.packed_wdt(wdown), _thr(threshold), out=output)


def _inner(input, wgate, wup, wdown, threshold, dtype):
    if input.dtype != dtype:
        raise RuntimeError(f"flash_gemv: this entry point expects {dtype} tensors, got {input.dtype}")
    if _dense_batch(input, wgate, wdown):
        return ops.mlp_dense(input, wgate, wup, wdown, _thr(threshold))
    return ops.mlp(input, wgate, wup, ops.packed_wdt(wdown), _thr(threshold))


def flag_gemv_gemv_inner(input, wgate, wup, wdown, threshold):
    """fp16 CATS MLP for decode; returns a new tensor shaped like ``input``; wdown is (H, I).
    Reference: flash_gemv.py:36-37, fuse_gemv_cmp_cuda.cu:2330-2405."""
    return _inner(input, wgate, wup, wdown, threshold, torch.float16)


def flag_gemv_gemv_inner_fp32(input, wgate, wup, wdown, threshold):
    """fp32 variant.  Reference: flash_gemv.py:39-40, fuse_gemv_cmp_cuda.cu:2407-2482."""
    return _inner(input, wgate, wup, wdown, threshold, torch.float32)


def flag_gemv_gemv_inner_bf16(input, wgate, wup, wdown, threshold):
    """bf16 variant.  Reference: flash_gemv.py:42-43, fuse_gemv_cmp_cuda.cu:2484-2560."""
    return _inner(input, wgate, wup, wdown, threshold, torch.bfloat16)


# ---- the names the reference implements with Triton --------------------------------------------
def gemv_gemv_triton(x, x_1, Wup, Wdownt, threshold):
    """CATS MLP from a precomputed x_1 = SiLU(gate_proj(x)): flags = |x_1| > threshold, then the
    masked up projection times x_1 and the masked transposed down projection.  Wup, Wdownt are
    (I, H).  Reference: flash_gemv/flash_gemv/__init__.py:45-48, kernels.py:45-462."""
    _, H = ops.batch_of(x)
    ws = ops.compact(x_1, None, _thr(threshold), H)
    return ops.updown(x, Wup, Wdownt, ws)


def flag_gemv_gemv_triton(x, Wgate, Wup, Wdownt, threshold):
    """As gemv_gemv_triton but computes the gate itself; Wgate is (H, I) (used as x @ Wgate).
    Reference: flash_gemv/flash_gemv/__init__.py:38-43."""
    return ops.mlp(x, ops.packed_wdt(Wgate), Wup, Wdownt, _thr(threshold))


def flag_gemv_gemv_dejavu(x, Wgate, Wup, Wdownt, threshold):
    """Index-list baseline of the reference (x is 2-D (1, H)); same result, same kernels here.
    Reference: flash_gemv/flash_gemv/__init__.py:50-54, kernels.py:464-1094."""
    return ops.mlp(x, ops.packed_wdt(Wgate), Wup, Wdownt, _thr(threshold))


def flag_gemv_gemv_fuse_dejavu(x, Wgate, Wup, Wdownt, threshold):
    """Reference: flash_gemv/flash_gemv/__init__.py:56-60, kernels.py:1096-1334."""
    return ops.mlp(x, ops.packed_wdt(Wgate), Wup, Wdownt, _thr(threshold))


# ---- torch.ops.flash_gemv.* ---------------------------------------------------------------------
# The reference registers its C++ functions with TORCH_LIBRARY(flash_gemv, m)
# (flash_gemv/csrc/fuse_gemv_cmp.cpp:87-102); the same operator names are registered here so code
# that calls torch.ops.flash_gemv.<op> directly keeps working.
_SCHEMAS = {
    "fuse_gemv_cmp": "(Tensor input, Tensor weight, Tensor(a!) output, Tensor(b!) idx, float threshold) -> int",
    "fuse_gemv_flag": "(Tensor input, Tensor weight, Tensor(a!) output, Tensor(b!) flag, float threshold) -> ()",
    "fuse_gemv_flag_gemv": "(Tensor input, Tensor wgate, Tensor wup, Tensor(a!) output, Tensor(b!) flag, float threshold) -> ()",
    "fuse_gemv_flag_gemv_gemv": "(Tensor input, Tensor wgate, Tensor wup, Tensor wdown, Tensor(a!) output, Tensor(b!) flag, float threshold) -> ()",
    "fuse_gemv_gemv_gemv": "(Tensor input, Tensor wgate, Tensor wup, Tensor wdown, Tensor(a!) output, float threshold) -> ()",
    "fuse_gemv_flag_batch": "(Tensor input, Tensor weight, Tensor(a!) output, Tensor(b!) flag, float threshold) -> ()",
    "fuse_gemv_flag_local": "(Tensor input, Tensor weight, Tensor(a!) output, Tensor(b!) flag, float threshold) -> ()",
    "fuse_flag_gemv_local": "(Tensor input, Tensor weight, Tensor(a!) output, Tensor flag) -> ()",
    "atomic_gemv": "(Tensor input, Tensor weight, Tensor(a!) output, Tensor flag) -> ()",
    "flag_gemv_gemv_atomic": "(Tensor input, Tensor wgate, Tensor wup, Tensor wdown, Tensor(a!) output, float threshold) -> ()",
    "flag_gemv_gemv": "(Tensor input, Tensor wgate, Tensor wup, Tensor wdown, Tensor(a!) output, float threshold) -> ()",
    "flag_gemv_gemv_inner": "(Tensor input, Tensor wgate, Tensor wup, Tensor wdown, float threshold) -> Tensor",
    "flag_gemv_gemv_inner_fp32": "(Tensor input, Tensor wgate, Tensor wup, Tensor wdown, float threshold) -> Tensor",
    "flag_gemv_gemv_inner_bf16": "(Tensor input, Tensor wgate, Tensor wup, Tensor wdown, float threshold) -> Tensor",
}
_torch_lib = None


def register_torch_ops() -> None:
    """Define ``torch.ops.flash_gemv.*`` (idempotent).  CUDA dispatch key only: calling an op with
    CPU tensors fails in the dispatcher — there is deliberately no CPU implementation."""
    global _torch_lib
    if _torch_lib is not None:
        return
    lib = torch.library.Library("flash_gemv", "DEF")
    g = globals()
    for name, schema in _SCHEMAS.items():
        lib.define(name + schema)
        lib.impl(name, g[name], "CUDA")
    _torch_lib = lib
