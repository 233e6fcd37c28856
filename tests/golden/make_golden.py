"""Generate tests/golden/*.npz by running the REFERENCE's own module on small seeded inputs.

Run it where a checkout of the reference (ScalingIntelligence/CATS) is available, with its path
in $CATS_REFERENCE:

    CATS_REFERENCE=<path to the CATS checkout> python tests/golden/make_golden.py

The reference module (experiments/models/sparse_silu/ugly_utils.py) imports plotting, training
and kernel packages that the decode path never touches (matplotlib, seaborn, peft, trl and the
un-built flash_gemv extension).  They are replaced by empty stand-in modules *after*
transformers has been imported, which is enough for ``import ugly_utils`` to succeed; the classes
exercised below (``LlamaSparseSiluMLP``, ``MistralSparseSiluMLP``, ``SparseSiLU``,
``get_threshold``) then run unmodified on the CPU.

The files hold inputs and the reference's outputs as float32/float64/bool arrays (16-bit cases
store the exactly representable values), under 2 MB in total.  The tests never need the
reference itself.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("CATS_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(HERE)), "..", "reference"))


def import_reference():
    import transformers  # noqa: F401  (must come before the stand-ins)
    from transformers import Trainer, TrainerCallback  # noqa: F401

    for name in ["matplotlib", "matplotlib.pyplot", "peft", "trl", "seaborn", "flash_gemv"]:
        if name not in sys.modules:
            sys.modules[name] = types.ModuleType(name)
    sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]
    sys.modules["peft"].PeftModel = object
    sys.modules["trl"].SFTTrainer = object
    sys.path.insert(0, REF)
    import experiments.models.sparse_silu.ugly_utils as U

    return U


def make_mlp(U, family, H, I, dtype, seed, wscale):
    from transformers import LlamaConfig, MistralConfig

    if family == "llama":
        cfg = LlamaConfig(hidden_size=H, intermediate_size=I, num_hidden_layers=1,
                          num_attention_heads=4, vocab_size=32)
        mlp = U.LlamaSparseSiluMLP(cfg)
    else:
        cfg = MistralConfig(hidden_size=H, intermediate_size=I, num_hidden_layers=1,
                            num_attention_heads=4, num_key_value_heads=2, vocab_size=32)
        mlp = U.MistralSparseSiluMLP(cfg)
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for lin in (mlp.gate_proj, mlp.up_proj, mlp.down_proj):
            lin.weight.copy_(torch.randn(lin.weight.shape, generator=g) * wscale)
    return mlp.to(dtype)


def f32(t):
    return t.detach().to(torch.float32).numpy()


def mlp_cases(U):
    """sp_method == 0 decode branch, prefill branch and the non-profile kill path."""
    out = {}
    specs = [
        # name, family, H, I, B, T, dtype, threshold, wscale
        ("llama_f32_b1", "llama", 64, 96, 1, 1, torch.float32, 0.10, 0.2),
        ("llama_f32_b3", "llama", 64, 96, 3, 1, torch.float32, 0.15, 0.2),
        ("llama_f32_odd", "llama", 264, 100, 2, 1, torch.float32, 0.05, 0.1),
        ("llama_f32_prefill", "llama", 64, 96, 2, 5, torch.float32, 0.10, 0.2),
        ("llama_f32_t0", "llama", 64, 96, 1, 1, torch.float32, 0.0, 0.2),
        ("llama_f32_tall", "llama", 64, 96, 1, 1, torch.float32, 1e9, 0.2),
        ("llama_f32_tneg", "llama", 64, 96, 2, 1, torch.float32, -1.0, 0.2),
        ("mistral_f32_b1", "mistral", 64, 160, 1, 1, torch.float32, 0.12, 0.15),
        ("mistral_f32_b4", "mistral", 64, 160, 4, 1, torch.float32, 0.20, 0.15),
        ("mistral_bf16_b2", "mistral", 64, 160, 2, 1, torch.bfloat16, 0.12, 0.15),
        ("llama_f16_b1", "llama", 64, 96, 1, 1, torch.float16, 0.10, 0.2),
        ("llama_f32_big", "llama", 128, 344, 1, 1, torch.float32, 0.07, 0.1),
    ]
    for k, (name, fam, H, I, B, T, dt, thr, ws) in enumerate(specs):
        mlp = make_mlp(U, fam, H, I, dt, seed=100 + k, wscale=ws)
        g = torch.Generator().manual_seed(900 + k)
        x = torch.randn(B, T, H, generator=g)
        x = (x / x.pow(2).mean(-1, keepdim=True).sqrt()).to(dt)
        mlp.is_profile = True
        mlp.sp_method = 0
        mlp.dead_threshold = thr
        with torch.no_grad():
            y_profile = mlp(x)
            # non-profile path with kill_sparse_swish_outputs (the path training/eval uses)
            mlp.is_profile = False
            mlp.kill_sparse_swish_outputs = True
            mlp.use_sparse_regularization = False
            y_kill = mlp(x)
            post = torch.nn.functional.silu(mlp.gate_proj(x))
            # given-mask branch (forward(x, sp_mask))
            sp_mask = (torch.rand(B, T, I, generator=g) > 0.3).to(dt)
            mlp.sparse_act_fn.set_new_threshold(thr)
            y_mask = mlp(x, sp_mask)
        out[name] = dict(
            family=fam, dtype=str(dt).replace("torch.", ""), threshold=np.float64(thr),
            x=f32(x), wg=f32(mlp.gate_proj.weight), wu=f32(mlp.up_proj.weight),
            wd=f32(mlp.down_proj.weight), y=f32(y_profile), y_kill=f32(y_kill),
            post_act=f32(post), sp_mask=f32(sp_mask), y_spmask=f32(y_mask),
        )
    return out


def activation_cases(U):
    g = torch.Generator().manual_seed(7)
    a = torch.randn(4, 257, generator=g) * 2
    out = {}
    for i, thr in enumerate([0.0, 0.05, 0.3, 1.0]):
        act = U.SparseSiLU(thr)
        out[f"sparse_silu_{i}"] = dict(a=f32(a), threshold=np.float64(thr), y=f32(act(a)))
    return out


def threshold_cases(U, mlp_cls_factory):
    """get_threshold on histograms collected by the reference's own collect_stats."""
    out = {}
    mlp = mlp_cls_factory()
    g = torch.Generator().manual_seed(11)
    pre = torch.randn(64, 96, generator=g) * 1.3
    post = torch.nn.functional.silu(pre)
    mlp.collect_stats(pre, post)
    bins = mlp.histogram_bins.clone()
    for i, s in enumerate([0.1, 0.3, 0.5, 0.7, 0.9]):
        counts = mlp.post_act_hist_counts.clone()
        thr = U.get_threshold(bins, counts.clone(), s)
        out[f"get_threshold_{i}"] = dict(bins=bins.numpy().astype(np.float64),
                                         counts=counts.numpy().astype(np.float64),
                                         pre_counts=mlp.pre_act_hist_counts.numpy().astype(np.float64),
                                         sparsity=np.float64(s), threshold=np.float64(float(thr)),
                                         pre=f32(pre), post=f32(post))
    return out


def main():
    torch.manual_seed(0)
    torch.set_num_threads(1)
    U = import_reference()
    cases = {}
    cases.update(mlp_cases(U))
    cases.update(activation_cases(U))
    cases.update(threshold_cases(U, lambda: make_mlp(U, "llama", 64, 96, torch.float32, 5, 0.2)))
    total = 0
    for name, arrays in cases.items():
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        total += os.path.getsize(path)
    print(f"wrote {len(cases)} golden files, {total / 1024:.0f} KiB, torch {torch.__version__}")


if __name__ == "__main__":
    main()
