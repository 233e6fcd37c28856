"""CATS MLP module with the reference's interface, running decode on the sm_100a kernels.

Mirrors the inference-relevant part of experiments/models/sparse_silu/ugly_utils.py:
``SparseSiLU`` (:80-92), ``{Llama,Mistral}SparseSiluMLP`` (:469-622, :807-959) with the same
constructor keywords, attributes (``is_profile``, ``sp_method``, ``dead_threshold``, ``wdown_t``,
``kill_sparse_swish_outputs``, ``use_relu``, ``is_stats`` ...) and ``forward(x, sp_mask=None)``,
and the model-level helpers the reference's bench scripts call (``apply_sparse_silu_mlp``,
``enable_sparse_silu``, ``activate_stats``, ``load_act_hist``, ``set_sparse_threshold``, ...;
experiments/bench_sparse_inference_llama.py:38-77), and the model-level classes those scripts
build their models from: ``get_sparse_config`` (:95-116), ``SparseLlamaConfig`` /
``SparseLlamaForCausalLM`` (:771-804), ``SparseMistralConfig`` / ``SparseMistralforCausalLM``
(:732-768) - so ``from cats_b200.sparse_silu import *`` gives a bench script every name it
takes from ``ugly_utils`` (``torch`` included, which the scripts use without importing it).

Dispatch of ``forward`` when ``is_profile`` is set (as in the reference, :877-904):
  decode (x.shape[1] == 1), sp_method 1 or 2 -> the CUDA path (``ops.mlp``); the reference calls
        flash_gemv.flag_gemv_gemv_inner_bf16 / gemv_gemv_triton here
  decode, sp_method 0                         -> dense thresholded PyTorch (the reference's own
        comparison branch, kept verbatim as the in-module reference)
  prefill (x.shape[1] > 1)                    -> dense thresholded PyTorch
The training-time extras of the reference module (regularisation terms, trainer callbacks, SVD
predictor) are not part of the decode path and are not reproduced.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn as nn
from . import ops

MISTRAL = "mistral"   # model_type strings of the reference's utils/constants.py
LLAMA = "llama"


class SparseSiLU(nn.SiLU):
    """SiLU whose outputs with |v| <= threshold are zeroed (ugly_utils.py:80-92)."""

    def __init__(self, threshold):
        super().__init__()
        self.threshold = threshold
        self.m = nn.Threshold(self.threshold, 0)

    def set_new_threshold(self, threshold):
        self.threshold = threshold
        self.m = nn.Threshold(threshold, 0)

    def forward(self, x):
        act = super().forward(x)
        return self.m(act) - self.m(-act)


def _cfg(config, name, default=None):
    if isinstance(config, dict):
        return config.get(name, default)
    return getattr(config, name, default)


class CatsSparseSiluMLP(nn.Module):
    """SiLU-gated MLP with CATS thresholding.  ``config`` needs ``hidden_size`` and
    ``intermediate_size`` (an HF LlamaConfig / MistralConfig or a dict)."""

    def __init__(self, config, *args, **kwargs):
        super().__init__()
        self.config = config
        self.hidden_size = _cfg(config, "hidden_size")
        self.intermediate_size = _cfg(config, "intermediate_size")
        self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.down_proj = nn.Linear(self.intermediate_size, self.hidden_size, bias=False)
        self.act_fn = nn.SiLU()

        self.swish_outputs = None
        self.relu = nn.ReLU()
        self.is_profile = False
        self.sp_method = 1
        self.wdown_t = None

        self.kill_sparse_swish_outputs = False
        self.dead_percentage = 0
        self.is_stats = False
        self.visit_counts = 0

        self.dead_threshold = kwargs.pop("dead_threshold", 0)
        self.use_sparse_regularization = kwargs.pop("use_sparse_regularization", True)
        self.regularization_type = kwargs.pop("regularization_type", "L1 regularization")
        self.regularization_threshold = kwargs.pop("regularization_threshold", 0.5)
        self.use_relu = kwargs.pop("use_relu", False)
        self.activation_norm = None

        # activation histograms: 1000 edges = -inf, 998 points on [-1, 1], +inf (ugly_utils.py:826-833)
        self.is_collect_histogram = False
        # (float32 CPU tensors whatever default device / dtype the model is being built under)
        num_bins = 1000
        f32 = dict(dtype=torch.float32, device="cpu")
        bins = torch.linspace(-1, 1, num_bins - 2, **f32)
        self.histogram_bins = torch.cat([torch.tensor([-torch.inf], **f32), bins,
                                         torch.tensor([torch.inf], **f32)])
        self._dev_hist = {}     # device -> (edges, pre counts, post counts): int64, on that device
        self.pre_act_hist_counts = torch.zeros(num_bins - 1, **f32)
        self.abs_post_act_hist_counts = torch.zeros(num_bins - 1, **f32)
        self.post_act_hist_counts = torch.zeros(num_bins - 1, **f32)
        self.t = 0
        self.count = 0
        self.agg_sparsity = 0

        self.sparse_act_fn = SparseSiLU(threshold=self.dead_threshold)

    # ---- statistics ---------------------------------------------------------------------------
    # The reference keeps the two histograms as float32 CPU tensors and fills them with
    # torch.histogram after copying the activations to the host on every forward
    # (ugly_utils.py:514-522).  Here CUDA activations are binned where they are (cats_histogram,
    # exact 64-bit counts per device); the counts are folded into the float32 CPU tensors of the
    # reference's format whenever those are read.
    def _fold_device_counts(self):
        for dev, (edges, pre, post) in list(self.__dict__.get("_dev_hist", {}).items()):
            self._pre_counts += pre.cpu().to(torch.float32)
            self._post_counts += post.cpu().to(torch.float32)
            pre.zero_()
            post.zero_()

    @property
    def pre_act_hist_counts(self):
        self._fold_device_counts()
        return self._pre_counts

    @pre_act_hist_counts.setter
    def pre_act_hist_counts(self, value):
        self._pre_counts = value

    @property
    def post_act_hist_counts(self):
        self._fold_device_counts()
        return self._post_counts

    @post_act_hist_counts.setter
    def post_act_hist_counts(self, value):
        self._post_counts = value

    def activate_stats(self, is_collect_histogram: bool = True):
        self.is_stats = True
        self.dead_percentage = 0
        self.visit_counts = 0
        self.is_collect_histogram = is_collect_histogram
        self.histogram_counts = torch.zeros(2000, dtype=torch.float32, device="cpu")

    def deactivate_stats(self):
        self.is_stats = False

    def collect_stats(self, pre_activation, post_activation):
        if pre_activation.is_cuda and post_activation.is_cuda:
            dev = pre_activation.device
            if dev not in self._dev_hist:
                n = self.histogram_bins.numel() - 1
                self._dev_hist[dev] = (self.histogram_bins.to(dev, torch.float32).contiguous(),
                                       torch.zeros(n, dtype=torch.int64, device=dev),
                                       torch.zeros(n, dtype=torch.int64, device=dev))
            edges, pre_counts, post_counts = self._dev_hist[dev]
            ops.histogram(pre_activation.detach().contiguous(), edges, pre_counts)
            ops.histogram(post_activation.detach().contiguous(), edges, post_counts, take_abs=True)
            return
        pre_activation = pre_activation.float().cpu().detach()
        post_activation = post_activation.float().cpu().detach()
        self.pre_act_hist_counts += torch.histogram(pre_activation, bins=self.histogram_bins)[0]
        self.post_act_hist_counts += torch.histogram(torch.abs(post_activation),
                                                     bins=self.histogram_bins)[0]

    # ---- forward ------------------------------------------------------------------------------
    def _dense_thresholded(self, x):
        post_act = self.act_fn(self.gate_proj(x))
        dead_neurons = post_act.abs() <= self.dead_threshold
        post_act[dead_neurons] = 0
        return self.down_proj(post_act * self.up_proj(x))

    def packed_down(self) -> torch.Tensor:
        """down_proj.weight as WdT (I, H).  Uses ``wdown_t`` when the caller set it the way the
        reference bench does (bench_sparse_inference_llama.py:76), else packs and caches."""
        w = self.wdown_t
        if w is not None and w.is_contiguous() and w.device == self.down_proj.weight.device:
            return w
        return ops.packed_wdt(self.down_proj.weight)

    def _cuda_decode(self, x):
        """The decode call, ~32 times per token under HF ``generate``: the validated launch state
        (weights, packed WdT, workspace, argument list) is kept per module and reused while
        nothing it depends on has changed; a call then costs one output allocation and one
        C call."""
        st = self.__dict__.get("_launch")
        wg, wu, wd = self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight
        key = (x.shape, x.dtype, x.device, wg.data_ptr(), wu.data_ptr(), wd.data_ptr(),
               wd._version, id(self.wdown_t), torch.cuda.current_stream(x.device).cuda_stream
               if x.is_cuda else 0)
        if st is None or st[0] != key or not x.is_contiguous():
            B, H = ops.batch_of(x)
            I = wg.shape[0]
            # batches: density-aware switch to the dense tensor-core path, which reads
            # down_proj.weight as it is (H, I); else the sparse kernels on the packed WdT (I, H)
            if (ops.use_dense(B, self.__dict__.get("sparsity_level")) and x.is_cuda
                    and wd.is_contiguous() and ops.dense_supported(B, H, I, x.dtype)):
                ops._req(x, "input")
                for w, name in ((wg, "gate weight"), (wu, "up weight"), (wd, "down weight")):
                    ops._req(w, name, x.dtype, x.device)
                fn, wdt, dev, dt = ops._lib.lib().cats_mlp_dense, wd, x.device, x.dtype
            else:
                wdt = self.packed_down()
                dev, dt, B, H, I = ops._check_mlp_weights(x, wg, wu, wdt)      # raises on misuse
                fn = ops._lib.lib().cats_mlp
            ws = ops.get_workspace(dev, H, I)
            st = (key, fn, wdt, ws, B, H, I, ops.dtype_code(dt), dev)
            self.__dict__["_launch"] = st
        _, fn, wdt, ws, B, H, I, code, dev = st
        out = torch.empty_like(x)
        with ops._on(dev):
            status = fn(x.data_ptr(), wg.data_ptr(), wu.data_ptr(), wdt.data_ptr(), ws.ptr, ws.nbytes,
                        B, H, I, code, float(self.dead_threshold), out.data_ptr(), ops.OUT_STORE,
                        None, None, None, 1e-6, key[-1])
        if status:
            ops._lib.check(status, "cats_mlp")
        return out

    def forward(self, x, sp_mask: Optional[torch.Tensor] = None):
        if sp_mask is not None:
            return self.down_proj(self.sparse_act_fn(self.gate_proj(x) * sp_mask) * self.up_proj(x))

        if self.is_profile:
            if x.shape[1] == 1 and self.sp_method in (1, 2):
                return self._cuda_decode(x)
            return self._dense_thresholded(x)

        if self.use_relu:
            post_act = self.relu(self.gate_proj(x))
            self.count += 1
            if self.is_stats:
                dead_neurons = post_act == 0
                dead_percentage = dead_neurons.float().mean()
                agg_sparsity = dead_neurons.all(dim=0).float().mean()
                self.dead_percentage = (self.dead_percentage * self.visit_counts + dead_percentage) / (
                    self.visit_counts + 1)
                self.agg_sparsity = (self.agg_sparsity * self.visit_counts + agg_sparsity) / (
                    self.visit_counts + 1)
                self.visit_counts += 1
            return self.down_proj(post_act * self.up_proj(x))

        self.count += 1
        pre_act = self.gate_proj(x)
        post_act = self.act_fn(pre_act)
        if self.kill_sparse_swish_outputs:
            dead_neurons = post_act.abs() <= self.dead_threshold
            dead_percentage = dead_neurons.float().mean()
            agg_sparsity = dead_neurons.all(dim=0).float().mean()
            if self.is_stats:
                self.dead_percentage = (self.dead_percentage * self.visit_counts + dead_percentage) / (
                    self.visit_counts + 1)
                self.agg_sparsity = (self.agg_sparsity * self.visit_counts + agg_sparsity) / (
                    self.visit_counts + 1)
                self.visit_counts += 1
                self.a = dead_percentage
                if self.is_collect_histogram and self._collect_this(pre_act):
                    self.collect_stats(pre_act, post_act)
            post_act[dead_neurons] = 0
        return self.down_proj(post_act * self.up_proj(x))

    def _collect_this(self, pre_act) -> bool:
        return True


class LlamaSparseSiluMLP(CatsSparseSiluMLP):
    """Reference: ugly_utils.py:807-959."""


class MistralSparseSiluMLP(CatsSparseSiluMLP):
    """Reference: ugly_utils.py:469-622 (skips histogram collection on all-padding batches)."""

    def _collect_this(self, pre_act) -> bool:
        return bool(pre_act.eq(0).float().mean() < 0.99)


# ---- model-level helpers (the reference's bench scripts import these with `import *`) ----------
def _layers(model):
    return model.model.layers


def get_model_type(model) -> str:
    """MISTRAL or LLAMA from the model's class name - the reference's rule
    (utils/utils.py:11-22): "mistral" is looked for first, then "llama"."""
    name = model.__class__.__name__.lower()
    if MISTRAL in name:
        return MISTRAL
    if LLAMA in name:
        return LLAMA
    raise ValueError(f"Model name {name} is not recognized.")


def get_mlp_class(model):
    """Mistral models get MistralSparseSiluMLP, Llama models LlamaSparseSiluMLP
    (ugly_utils.py:64-66)."""
    return MistralSparseSiluMLP if get_model_type(model) == MISTRAL else LlamaSparseSiluMLP


def apply_sparse_silu_mlp(model, config, use_sparse_regularization: bool = False):
    """Swap every layer's MLP for the CATS module, sharing the three nn.Linear layers
    (ugly_utils.py:119-131)."""
    SparseMLP = get_mlp_class(model)
    for layer in _layers(model):
        original_mlp = layer.mlp
        new_mlp = SparseMLP(config, use_sparse_regularization=use_sparse_regularization)
        new_mlp.gate_proj = original_mlp.gate_proj
        new_mlp.up_proj = original_mlp.up_proj
        new_mlp.down_proj = original_mlp.down_proj
        layer.mlp = new_mlp


def _sparse_mlps(model):
    for i, layer in enumerate(_layers(model)):
        if isinstance(layer.mlp, CatsSparseSiluMLP):
            yield i, layer.mlp


def activate_stats(model, is_collect_histogram: bool = True):
    for _, mlp in _sparse_mlps(model):
        mlp.activate_stats(is_collect_histogram=is_collect_histogram)


def deactivate_stats(model):
    for _, mlp in _sparse_mlps(model):
        mlp.deactivate_stats()


def enable_sparse_silu(model):
    for _, mlp in _sparse_mlps(model):
        mlp.kill_sparse_swish_outputs = True


def disable_sparse_silu(model):
    for _, mlp in _sparse_mlps(model):
        mlp.kill_sparse_swish_outputs = False


def print_dead_neuron_stats(model):
    total, sparsity_list = 0.0, []
    for i, mlp in _sparse_mlps(model):
        dead = float(mlp.dead_percentage) * 100
        sparsity_list.append(dead)
        total += dead
        print(f"layer {i} sparsity: {dead:.3f}%  agg sparsity: {float(mlp.agg_sparsity) * 100:.3f}%")
    mean = total / max(1, len(sparsity_list))
    print(f"Total sparsity: {mean: .3f}%")
    return mean, sparsity_list


def get_threshold(bin_edges: torch.Tensor, histogram_counts: torch.Tensor, sparsity_level: float):
    """Bin edge at which the normalised histogram's CDF crosses ``sparsity_level``
    (ugly_utils.py:236-245; note that, as there, the counts tensor is normalised in place)."""
    assert len(bin_edges.shape) == len(histogram_counts.shape) == 1, \
        "bin_edges and histogram are expected to be 1-dimensional."
    histogram_counts /= histogram_counts.sum()
    threshold_idx = torch.searchsorted(histogram_counts.cumsum(0), sparsity_level, side="right")
    return bin_edges[threshold_idx]


def set_sparse_threshold(model, sparsity_level: float, use_relu: bool = False):
    """Per-layer threshold from the collected |post-activation| histogram (ugly_utils.py:257-273)."""
    for _, mlp in _sparse_mlps(model):
        if not mlp.is_stats:
            continue
        if use_relu:
            mlp.sparse_act_fn = nn.ReLU()
            mlp.use_relu = True
        else:
            mlp.dead_threshold = get_threshold(mlp.histogram_bins, mlp.post_act_hist_counts,
                                               sparsity_level)
            mlp.sparsity_level = sparsity_level      # hint for the batch path switch
            mlp.sparse_act_fn.set_new_threshold(mlp.dead_threshold)
            mlp.regularization_threshold = mlp.dead_threshold * 1.2


def save_act_hist(model, filename: str):
    """{layer: (bins, pre_counts, post_counts)} via torch.save (ugly_utils.py:399-413)."""
    os.makedirs(os.path.dirname(filename) or ".", exist_ok=True)
    act_dict = {}
    for i, mlp in _sparse_mlps(model):
        if mlp.is_stats:
            act_dict[i] = (mlp.histogram_bins, mlp.pre_act_hist_counts, mlp.post_act_hist_counts)
    torch.save(act_dict, filename)


def load_act_hist(model, filename: str):
    """Inverse of save_act_hist; reads the reference's histogram files (ugly_utils.py:416-433)."""
    assert os.path.exists(filename), f"{filename} does not exist when loading the activation histogram."
    act_dict = torch.load(filename)
    for i, mlp in _sparse_mlps(model):
        if mlp.is_stats:
            mlp.histogram_bins, mlp.pre_act_hist_counts, mlp.post_act_hist_counts = act_dict[i]



# ---- model-level classes (cats_b200/sparse_models.py), imported on first use --------------------
# They subclass the HF Llama / Mistral models, and importing those takes seconds, which the
# operator-level users of this module should not pay.  ``__all__`` lists them, so
# ``from cats_b200.sparse_silu import *`` still delivers every name (that is what triggers the
# import then).
_MODEL_NAMES = ("get_sparse_config", "SparseLlamaConfig", "SparseLlamaForCausalLM",
                "SparseMistralConfig", "SparseMistralforCausalLM")

__all__ = [
    "torch", "nn", "os", "MISTRAL", "LLAMA", "SparseSiLU", "CatsSparseSiluMLP",
    "LlamaSparseSiluMLP", "MistralSparseSiluMLP", "get_model_type", "get_mlp_class", "apply_sparse_silu_mlp",
    "activate_stats", "deactivate_stats", "enable_sparse_silu", "disable_sparse_silu",
    "print_dead_neuron_stats", "get_threshold", "set_sparse_threshold", "save_act_hist",
    "load_act_hist", *_MODEL_NAMES,
]


def __getattr__(name):
    if name in _MODEL_NAMES:
        from . import sparse_models

        return getattr(sparse_models, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
