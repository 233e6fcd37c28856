"""The lean decode loop (cats_b200/decoder.py) against HF's own forward, on CPU with tiny models:
prefill logits, then single-token steps on the static KV cache, for the Llama (MHA) and Mistral
(GQA) layouts, with the dense MLP and with the dense thresholded MLP (the reference's
``sp_method = 0`` branch, which the HF model runs through the swapped-in CATS module)."""
import pytest
import torch

from cats_b200 import decoder as D
from cats_b200 import sparse_silu as S

TINY = dict(hidden_size=64, intermediate_size=160, num_hidden_layers=3, num_attention_heads=4,
            vocab_size=128, max_position_embeddings=512)


def tiny_model(family, thresholds=None):
    from transformers import LlamaConfig, MistralConfig

    torch.manual_seed(0)
    if family == "llama":
        cfg, cls, mt = LlamaConfig(**TINY, num_key_value_heads=4), S.SparseLlamaForCausalLM, S.LLAMA
    else:
        cfg = MistralConfig(**TINY, num_key_value_heads=2, sliding_window=None)
        cls, mt = S.SparseMistralforCausalLM, S.MISTRAL
    cfg = S.get_sparse_config(cfg, model_type=mt, use_sparse_model=True, thresholds=thresholds)
    cfg.use_relu = False
    model = cls(cfg).eval()
    with torch.no_grad():
        for p in model.parameters():      # HF's init is N(0, 0.02): too small to exercise anything
            if p.dim() == 2:
                p.normal_(0, 0.15)
    return model


@pytest.mark.parametrize("family", ["llama", "mistral"])
@pytest.mark.parametrize("mode", ["dense", "masked"])
def test_prefill_and_steps_match_the_hf_forward(family, mode):
    thr = [0.05, 0.1, 0.2] if mode == "masked" else None
    model = tiny_model(family, thr)
    if mode == "masked":
        for l in model.model.layers:          # HF forward -> CATS module -> dense thresholded
            l.mlp.is_profile, l.mlp.sp_method = True, 0
    else:
        S.disable_sparse_silu(model)
    B, T, n_new = 2, 9, 5
    ids = torch.randint(0, TINY["vocab_size"], (B, T))
    dec = D.CatsDecoder(model, batch=B, max_len=300, mlp=mode, thresholds=thr)
    with torch.no_grad():
        ref = model(ids, use_cache=False).logits
        logits = dec.prefill(ids)
        assert torch.allclose(logits, ref[:, -1], rtol=1e-4, atol=1e-4)
        seq = ids
        for step in range(n_new):
            nxt = dec.tok.clone()
            seq = torch.cat([seq, nxt[:, None]], 1)
            dec._step(D.BUCKET)
            ref = model(seq, use_cache=False).logits[:, -1]
            assert torch.allclose(dec.logits, ref, rtol=1e-4, atol=1e-4), step
            assert torch.equal(dec.tok, ref.argmax(-1))
        assert int(dec.pos) == T + n_new


def test_calibration_sets_a_threshold_per_layer_near_the_requested_sparsity():
    model = tiny_model("llama")
    thr = D.calibrate(model, 0.5, n_prompts=3, prompt_len=32)
    assert len(thr) == 3 and all(t > 0 for t in thr)
    x = torch.randn(64, TINY["hidden_size"])
    for l, t in zip(model.model.layers, thr):
        assert not l.mlp.is_stats and float(l.mlp.dead_threshold) == t
    # the first layer's input distribution is known (normalised embeddings): about half is dead
    l0 = model.model.layers[0]
    ids = torch.randint(0, TINY["vocab_size"], (1, 200))
    with torch.no_grad():
        h = l0.post_attention_layernorm(model.model.embed_tokens(ids))
        dead = (l0.mlp.act_fn(l0.mlp.gate_proj(h)).abs() <= thr[0]).float().mean()
    assert 0.3 < float(dead) < 0.7
