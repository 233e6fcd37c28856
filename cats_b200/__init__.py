"""cats_b200 — B200-native (sm_100a) CATS thresholded sparse-MLP decode path.

Layers, bottom up:
  csrc/ + include/cats_b200.h   hand-written CUDA kernels behind a C ABI (``libcats_b200.so``)
  _lib                          ctypes binding of that ABI
  ops                           torch-tensor front end (validation, workspaces, streams)
  flash_gemv                    the reference's ``flash_gemv`` operator API on top of ``ops``
  sparse_silu                   the reference's CATS MLP module interface on top of ``ops``
  synth                         seeded synthetic weights / inputs / thresholds for tests and benches
  tp                            intermediate-dimension sharding with one all-reduce per layer

Importing the package does not load CUDA; the first operator call does, and raises if the
library cannot be built or loaded (there is no CPU or PyTorch fallback).
"""
from . import flash_gemv, ops, sparse_silu  # noqa: F401
from ._lib import lib, lib_path  # noqa: F401

__version__ = "0.1.0"
