"""Model-level classes of the reference's CATS module, decode-relevant parts only.

``get_sparse_config`` (experiments/models/sparse_silu/ugly_utils.py:95-116), ``SparseLlamaConfig``
/ ``SparseLlamaForCausalLM`` (:771-804) and ``SparseMistralConfig`` / ``SparseMistralforCausalLM``
(:732-768): what experiments/bench_sparse_inference_{llama,mistral}.py:23-41 build their models
from.  The constructors re-apply ``config.thresholds`` as each layer's ``dead_threshold``
(:784-792), which is how a saved CATS checkpoint gets its thresholds back.  Reached through
``cats_b200.sparse_silu`` (which imports this module on first use of one of these names).
"""
from __future__ import annotations

from transformers import (LlamaConfig, LlamaForCausalLM, MistralConfig, MistralForCausalLM,
                          PretrainedConfig)

from .sparse_silu import (LLAMA, MISTRAL, CatsSparseSiluMLP, LlamaSparseSiluMLP,  # noqa: F401
                          MistralSparseSiluMLP, apply_sparse_silu_mlp)


class SparseLlamaConfig(LlamaConfig):
    """ugly_utils.py:771-775."""
    model_type = "sparse_llama"

    def __init__(self, **kwargs):
        super().__init__(**kwargs)


class SparseMistralConfig(MistralConfig):
    """ugly_utils.py:732-736."""
    model_type = "sparse_mistral"

    def __init__(self, **kwargs):
        super().__init__(**kwargs)


def get_sparse_config(config: PretrainedConfig, model_type: str = None, use_sparse_model=False,
                      use_sparse_predictor=False, use_sparse_regularization=False,
                      use_graceful_regularization=False, thresholds=None):
    """A Sparse{Llama,Mistral}Config carrying every field of ``config`` plus the CATS switches
    (ugly_utils.py:95-116).  ``thresholds``: per-layer list that the CausalLM classes re-apply."""
    new_config = SparseMistralConfig() if model_type == MISTRAL else SparseLlamaConfig()
    new_config.__dict__.update(config.__dict__)
    config = new_config
    config.use_sparse_model = use_sparse_model
    config.use_sparse_predictor = use_sparse_predictor
    config.use_sparse_regularization = use_sparse_regularization
    config.use_graceful_regularization = use_graceful_regularization
    config.thresholds = thresholds
    return config


def _apply_config_thresholds(model, mlp_class):
    """What both CausalLM constructors do after swapping the MLPs (ugly_utils.py:784-792, 745-753):
    thresholds saved in the config come back as ``dead_threshold`` with the sparse activation on."""
    config = model.config
    thresholds = getattr(config, "thresholds", None)
    if thresholds is None:
        return
    for idx, m in enumerate(model.model.layers):
        if isinstance(m.mlp, mlp_class):
            m.mlp.dead_threshold = thresholds[idx]
            m.mlp.sparse_act_fn.set_new_threshold(m.mlp.dead_threshold)
            m.mlp.kill_sparse_swish_outputs = True
            m.mlp.use_relu = getattr(config, "use_relu", False)


class _SparseCausalLMMixin:
    """Decode-relevant part of the reference's CausalLM subclasses.  The SVD sparsity predictor
    (``use_sparse_predictor``, ugly_utils.py:793-794) is a training-time component outside the
    decode path: asking for it raises instead of silently running without it."""
    _sparse_mlp_class = CatsSparseSiluMLP

    def _init_sparse(self, config):
        self.config = config
        if getattr(config, "use_sparse_model", False):
            self.apply_sparse_mlp()
            _apply_config_thresholds(self, self._sparse_mlp_class)
        if getattr(config, "use_sparse_predictor", False):
            self.apply_sparse_predictor(init_svd=getattr(config, "init_svd", True))

    def apply_sparse_mlp(self):
        apply_sparse_silu_mlp(self, config=self.config,
                              use_sparse_regularization=getattr(self.config, "use_sparse_regularization", False))

    def apply_sparse_predictor(self, init_svd: bool = True):
        raise RuntimeError("cats_b200: the SVD sparsity predictor of the reference is not part of "
                           "the decode path and is not provided")


class SparseLlamaForCausalLM(_SparseCausalLMMixin, LlamaForCausalLM):
    """ugly_utils.py:778-804."""
    config_class = SparseLlamaConfig
    _sparse_mlp_class = LlamaSparseSiluMLP

    def __init__(self, config):
        super().__init__(config)
        self._init_sparse(config)


class SparseMistralforCausalLM(_SparseCausalLMMixin, MistralForCausalLM):
    """ugly_utils.py:739-768 (the class name is spelt as in the reference)."""
    config_class = SparseMistralConfig
    _sparse_mlp_class = MistralSparseSiluMLP

    def __init__(self, config):
        super().__init__(config)
        self._init_sparse(config)
