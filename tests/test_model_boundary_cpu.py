"""The model-level boundary: what the reference's bench scripts take from ``ugly_utils`` with
``import *`` must come out of ``cats_b200.sparse_silu`` the same way.

The bodies below are the statements of ``prepare_sparse_model`` and of the set-up part of
``benchmark_decode`` (experiments/bench_sparse_inference_llama.py:23-41, 56-77 and the Mistral
twin), executed in a namespace filled by ``from cats_b200.sparse_silu import *``.  Stand-ins, all
named here: ``from_pretrained`` of a checkpoint directory becomes a tiny random-init config and
the plain constructor (there are no checkpoints offline); the tokenizer lines are dropped; the
activation-histogram file is one this test writes first with ``save_act_hist``.
"""
import os

import pytest
import torch

TINY = dict(hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
            vocab_size=128, max_position_embeddings=64)


def star_namespace():
    ns = {}
    exec("from cats_b200.sparse_silu import *", ns)
    return ns


def test_star_import_delivers_every_name_the_scripts_use():
    ns = star_namespace()
    for name in ("torch", "get_sparse_config", "apply_sparse_silu_mlp", "enable_sparse_silu",
                 "activate_stats", "load_act_hist", "set_sparse_threshold", "deactivate_stats",
                 "SparseLlamaConfig", "SparseLlamaForCausalLM", "SparseMistralConfig",
                 "SparseMistralforCausalLM", "LlamaSparseSiluMLP", "MistralSparseSiluMLP",
                 "SparseSiLU", "save_act_hist", "get_threshold", "print_dead_neuron_stats"):
        assert name in ns, name


PREPARE_LLAMA = """
BaseConfig = LlamaConfig
SparseConfig = SparseLlamaConfig
SparseCausalLM = SparseLlamaForCausalLM
SparseConfig.register_for_auto_class()
SparseCausalLM.register_for_auto_class("AutoModelForCausalLM")

config = BaseConfig(**TINY, num_key_value_heads=4)          # stand-in for from_pretrained
config = get_sparse_config(config)
config.use_cache = True
model = SparseCausalLM(config)                               # stand-in for from_pretrained
model.config_class = SparseConfig
apply_sparse_silu_mlp(model, model.config, use_sparse_regularization=False)
enable_sparse_silu(model)
model.config.use_sparse_predictor = False
model.config.use_relu = False
model.config.use_sparse_model = True
"""

PREPARE_MISTRAL = """
BaseConfig = MistralConfig
SparseConfig = MistralForCausalLM
SparseCausalLM = SparseMistralforCausalLM
SparseConfig.register_for_auto_class()
SparseCausalLM.register_for_auto_class("AutoModelForCausalLM")

config = BaseConfig(**TINY, num_key_value_heads=2)          # stand-in for from_pretrained
config = get_sparse_config(config)
config.use_cache = True
model = SparseCausalLM(config)                               # stand-in for from_pretrained
model.config_class = SparseConfig
apply_sparse_silu_mlp(model, model.config, use_sparse_regularization=False)
enable_sparse_silu(model)
model.config.use_sparse_predictor = False
model.config.use_relu = False
model.config.use_sparse_model = True
"""

SETUP = """
activate_stats(model)
load_act_hist(model, act_hist_path)
set_sparse_threshold(model, 0.5)
deactivate_stats(model)
for m in model.model.layers:
    m.mlp.is_profile = True
    # m.mlp.use_flash_gemv = True
    if method == 0:
        m.mlp.sp_method = 0
        print(m.mlp.down_proj.weight.dtype)
    elif method == 1:
        m.mlp.sp_method = 1
    elif method == 2:
        m.mlp.sp_method = 2
        m.mlp.wdown_t = m.mlp.down_proj.weight.t().contiguous()
        print(m.mlp.down_proj.weight.dtype)
model.eval()
"""


@pytest.mark.parametrize("family", ["llama", "mistral"])
@pytest.mark.parametrize("method", [0, 2])
def test_script_bodies_run_on_a_tiny_random_model(family, method, tmp_path):
    from transformers import LlamaConfig, MistralConfig, MistralForCausalLM

    ns = star_namespace()
    ns.update(TINY=TINY, LlamaConfig=LlamaConfig, MistralConfig=MistralConfig,
              MistralForCausalLM=MistralForCausalLM, method=method)
    torch.manual_seed(0)
    exec(PREPARE_LLAMA if family == "llama" else PREPARE_MISTRAL, ns)
    model = ns["model"]
    mlp_name = "LlamaSparseSiluMLP" if family == "llama" else "MistralSparseSiluMLP"
    assert all(type(l.mlp).__name__ == mlp_name for l in model.model.layers)
    assert all(l.mlp.kill_sparse_swish_outputs for l in model.model.layers)

    # the histogram file the script loads: collected here with the module's own statistics path
    ids = torch.randint(0, TINY["vocab_size"], (2, 24))
    ns["activate_stats"](model)
    with torch.no_grad():
        model(ids)
    path = os.path.join(tmp_path, "hist", "activation_histogram.pt")
    ns["save_act_hist"](model, path)
    ns["deactivate_stats"](model)
    ns["act_hist_path"] = path

    exec(SETUP, ns)
    for layer in model.model.layers:
        mlp = layer.mlp
        assert mlp.is_profile and mlp.sp_method == method and not mlp.is_stats
        assert float(mlp.dead_threshold) > 0            # a bin edge of the |post-act| histogram
        if method == 2:
            assert tuple(mlp.wdown_t.shape) == (TINY["intermediate_size"], TINY["hidden_size"])
    # prefill takes the dense thresholded branch on any device: about half the neurons are dead
    with torch.no_grad():
        logits = model(ids).logits
    assert logits.shape == (2, 24, TINY["vocab_size"]) and torch.isfinite(logits).all()
    mlp = model.model.layers[0].mlp
    x = torch.randn(4, 16, TINY["hidden_size"])
    dead = (mlp.act_fn(mlp.gate_proj(x)).abs() <= mlp.dead_threshold).float().mean()
    assert 0.2 < float(dead) < 0.8


def test_thresholds_in_the_config_come_back_as_dead_thresholds():
    """SparseLlamaForCausalLM.__init__ re-applies config.thresholds (ugly_utils.py:784-792): the
    way a saved CATS checkpoint gets its per-layer thresholds back."""
    from transformers import LlamaConfig, MistralConfig

    from cats_b200 import sparse_silu as S

    cfg = S.get_sparse_config(LlamaConfig(**TINY, num_key_value_heads=4), use_sparse_model=True,
                              thresholds=[0.125, 0.25])
    cfg.use_relu = False
    model = S.SparseLlamaForCausalLM(cfg)
    for t, layer in zip((0.125, 0.25), model.model.layers):
        assert isinstance(layer.mlp, S.LlamaSparseSiluMLP)
        assert layer.mlp.dead_threshold == t and layer.mlp.sparse_act_fn.threshold == t
        assert layer.mlp.kill_sparse_swish_outputs and layer.mlp.use_relu is False
    assert type(cfg).__name__ == "SparseLlamaConfig" and cfg.model_type == "sparse_llama"

    mc = S.get_sparse_config(MistralConfig(**TINY, num_key_value_heads=2), model_type=S.MISTRAL,
                             use_sparse_model=True, thresholds=[0.5, 0.75])
    mc.use_relu = False
    mm = S.SparseMistralforCausalLM(mc)
    assert [l.mlp.dead_threshold for l in mm.model.layers] == [0.5, 0.75]
    assert all(isinstance(l.mlp, S.MistralSparseSiluMLP) for l in mm.model.layers)
    assert type(mc).__name__ == "SparseMistralConfig"
    # no thresholds, no sparse model: a plain HF model
    plain = S.SparseLlamaForCausalLM(S.get_sparse_config(LlamaConfig(**TINY, num_key_value_heads=4)))
    assert not isinstance(plain.model.layers[0].mlp, S.CatsSparseSiluMLP)
    with pytest.raises(RuntimeError, match="predictor"):
        bad = S.get_sparse_config(LlamaConfig(**TINY, num_key_value_heads=4), use_sparse_predictor=True)
        S.SparseLlamaForCausalLM(bad)


def test_packed_down_weight_is_tied_to_the_live_tensor():
    """The cache of packed WdT copies must not hand a stale copy to a new weight that happens to
    get a freed weight's address (same shape, same version counter)."""
    from cats_b200 import ops

    calls = []
    real = ops.transpose
    ops.transpose = lambda w: (calls.append(1), w.t().contiguous())[1]
    saved_req = ops._req
    ops._req = lambda *a, **k: None        # CPU tensors stand in for CUDA ones in this test
    try:
        ops.clear_packed()
        w1 = torch.randn(8, 24)
        p1 = ops.packed_wdt(w1)
        assert ops.packed_wdt(w1) is p1 and len(calls) == 1
        addr = w1.data_ptr()
        del w1, p1
        import gc
        gc.collect()
        assert not ops._packed                      # the entry went away with the weight
        w2 = torch.randn(8, 24)
        for _ in range(50):                         # usually lands on the freed address at once
            if w2.data_ptr() == addr:
                break
            w2 = torch.randn(8, 24)
        p2 = ops.packed_wdt(w2)
        assert torch.equal(p2, w2.t()) and len(calls) == 2
        w2.add_(1.0)                                # in-place update: version counter moves
        assert torch.equal(ops.packed_wdt(w2), w2.t()) and len(calls) == 3
    finally:
        ops.transpose, ops._req = real, saved_req
        ops.clear_packed()
