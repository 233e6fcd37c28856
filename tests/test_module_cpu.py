"""Host-side mirror of the reference interface, checked on the CPU against the golden files:
the module's dense branches (prefill, sp_method 0, given mask, kill path), SparseSiLU,
get_threshold, histogram save/load, and the operator names."""
import inspect
import os

import numpy as np
import pytest
import torch

from conftest import MLP_GOLDEN, golden_names, load_golden
import cats_b200
from cats_b200 import flash_gemv as fg
from cats_b200 import sparse_silu as S
import flash_gemv as alias

DT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
# same torch calls as the reference; only the BLAS summation order (thread count) may differ
TOL = {"float32": 2e-6, "float16": 2e-3, "bfloat16": 2e-2}


def close(y, ref, dtype="float32"):
    y = y.float().numpy().astype(np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref)
    return np.linalg.norm(y - ref) <= TOL[dtype] * (den if den > 0 else 1.0)


def module_from_golden(g):
    H, I = g["wg"].shape[1], g["wg"].shape[0]
    cls = S.MistralSparseSiluMLP if str(g["family"]) == "mistral" else S.LlamaSparseSiluMLP
    m = cls({"hidden_size": H, "intermediate_size": I})
    dt = DT[str(g["dtype"])]
    with torch.no_grad():
        m.gate_proj.weight.copy_(torch.from_numpy(g["wg"]))
        m.up_proj.weight.copy_(torch.from_numpy(g["wu"]))
        m.down_proj.weight.copy_(torch.from_numpy(g["wd"]))
    m = m.to(dt)
    m.dead_threshold = float(g["threshold"])
    return m, torch.from_numpy(g["x"]).to(dt)


@pytest.mark.parametrize("name", MLP_GOLDEN)
def test_dense_branches_bit_match_reference(name):
    g = load_golden(name)
    m, x = module_from_golden(g)
    with torch.no_grad():
        m.is_profile, m.sp_method = True, 0
        dt = str(g["dtype"])
        y = m(x)
        assert close(y, g["y"], dt)
        m.is_profile = False
        m.kill_sparse_swish_outputs = True
        assert close(m(x), g["y_kill"], dt)
        m.sparse_act_fn.set_new_threshold(float(g["threshold"]))
        ym = m(x, torch.from_numpy(g["sp_mask"]).to(x.dtype))
        assert close(ym, g["y_spmask"], dt)


def test_prefill_takes_dense_branch_even_with_cuda_method():
    g = load_golden("llama_f32_prefill")
    m, x = module_from_golden(g)
    m.is_profile, m.sp_method = True, 1
    with torch.no_grad():
        assert close(m(x), g["y"])


def test_decode_on_cpu_raises_instead_of_falling_back():
    g = load_golden("llama_f32_b1")
    m, x = module_from_golden(g)
    m.is_profile, m.sp_method = True, 1
    with pytest.raises(RuntimeError, match="CUDA"):
        m(x)


@pytest.mark.parametrize("name", golden_names("sparse_silu_"))
def test_sparse_silu_module(name):
    g = load_golden(name)
    y = S.SparseSiLU(float(g["threshold"]))(torch.from_numpy(g["a"]))
    assert np.array_equal(y.numpy(), g["y"])


@pytest.mark.parametrize("name", golden_names("get_threshold_"))
def test_get_threshold_and_collect_stats(name):
    g = load_golden(name)
    m = S.LlamaSparseSiluMLP({"hidden_size": 64, "intermediate_size": 96})
    m.collect_stats(torch.from_numpy(g["pre"]), torch.from_numpy(g["post"]))
    assert np.array_equal(m.post_act_hist_counts.numpy().astype(np.float64), g["counts"])
    assert np.array_equal(m.pre_act_hist_counts.numpy().astype(np.float64), g["pre_counts"])
    t = S.get_threshold(m.histogram_bins, m.post_act_hist_counts.clone(), float(g["sparsity"]))
    assert float(t) == float(g["threshold"])


class _Layer(torch.nn.Module):
    def __init__(self, H, I):
        super().__init__()
        self.mlp = torch.nn.Module()
        self.mlp.gate_proj = torch.nn.Linear(H, I, bias=False)
        self.mlp.up_proj = torch.nn.Linear(H, I, bias=False)
        self.mlp.down_proj = torch.nn.Linear(I, H, bias=False)


class _ModelBase(torch.nn.Module):
    def __init__(self, H=64, I=96, L=2):
        super().__init__()
        self.config = type("Cfg", (), {"hidden_size": H, "intermediate_size": I})()
        self.model = torch.nn.Module()
        self.model.layers = torch.nn.ModuleList([_Layer(H, I) for _ in range(L)])


# the model family is read off the class name, as in the reference (utils/utils.py:11-22)
class TinyMistralForCausalLM(_ModelBase):
    pass


class TinyLlamaForCausalLM(_ModelBase):
    pass


def _Model(family, **kw):
    return (TinyMistralForCausalLM if family == "mistral" else TinyLlamaForCausalLM)(**kw)


def test_model_helpers_follow_the_bench_script_sequence(tmp_path):
    """apply -> enable -> activate_stats -> (forward) -> save/load hist -> set threshold, the
    sequence of experiments/bench_sparse_inference_llama.py:38-77."""
    model = _Model("mistral")
    lin = model.model.layers[0].mlp.gate_proj
    S.apply_sparse_silu_mlp(model, model.config)
    mlp0 = model.model.layers[0].mlp
    assert isinstance(mlp0, S.MistralSparseSiluMLP) and mlp0.gate_proj is lin
    assert S.get_mlp_class(_Model("llama")) is S.LlamaSparseSiluMLP
    S.enable_sparse_silu(model)
    S.activate_stats(model)
    x = torch.randn(3, 4, 64)
    with torch.no_grad():
        for layer in model.model.layers:
            layer.mlp(x)
    assert float(mlp0.post_act_hist_counts.sum()) == 3 * 4 * 96
    path = os.path.join(tmp_path, "hist.pt")
    S.save_act_hist(model, path)
    model2 = _Model("mistral")
    S.apply_sparse_silu_mlp(model2, model2.config)
    S.activate_stats(model2)
    S.load_act_hist(model2, path)
    S.set_sparse_threshold(model2, 0.5)
    S.deactivate_stats(model2)
    t = model2.model.layers[0].mlp.dead_threshold
    assert isinstance(t, torch.Tensor) and t.dim() == 0 and float(t) > 0
    for m in model2.model.layers:
        m.mlp.is_profile = True
        m.mlp.sp_method = 2
        m.mlp.wdown_t = m.mlp.down_proj.weight.t().contiguous()
    S.disable_sparse_silu(model2)
    assert not model2.model.layers[0].mlp.kill_sparse_swish_outputs


REFERENCE_SIGNATURES = {
    # flash_gemv/flash_gemv/flash_gemv.py:3-43 and __init__.py:38-60
    "fuse_gemv_cmp": ["input", "weight", "output", "idx", "threshold"],
    "fuse_gemv_flag": ["input", "weight", "output", "flag", "threshold"],
    "fuse_gemv_flag_gemv": ["input", "wgate", "wup", "output", "flag", "threshold"],
    "fuse_gemv_flag_gemv_gemv": ["input", "wgate", "wup", "wdown", "output", "flag", "threshold"],
    "fuse_gemv_gemv_gemv": ["input", "wgate", "wup", "wdown", "output", "threshold"],
    "fuse_gemv_flag_batch": ["input", "weight", "output", "flag", "threshold"],
    "fuse_gemv_flag_local": ["input", "weight", "output", "flag", "threshold"],
    "fuse_flag_gemv_local": ["input", "weight", "output", "flag"],
    "atomic_gemv": ["input", "weight", "output", "flag"],
    "flag_gemv_gemv_atomic": ["input", "wgate", "wup", "wdown", "output", "threshold"],
    "flag_gemv_gemv": ["input", "wgate", "wup", "wdown", "output", "threshold"],
    "flag_gemv_gemv_inner": ["input", "wgate", "wup", "wdown", "threshold"],
    "flag_gemv_gemv_inner_fp32": ["input", "wgate", "wup", "wdown", "threshold"],
    "flag_gemv_gemv_inner_bf16": ["input", "wgate", "wup", "wdown", "threshold"],
    "flag_gemv_gemv_triton": ["x", "Wgate", "Wup", "Wdownt", "threshold"],
    "gemv_gemv_triton": ["x", "x_1", "Wup", "Wdownt", "threshold"],
    "flag_gemv_gemv_fuse_dejavu": ["x", "Wgate", "Wup", "Wdownt", "threshold"],
    "flag_gemv_gemv_dejavu": ["x", "Wgate", "Wup", "Wdownt", "threshold"],
}


def test_operator_api_names_and_arguments():
    assert sorted(fg.__all__) == sorted(REFERENCE_SIGNATURES)
    for name, args in REFERENCE_SIGNATURES.items():
        for mod in (fg, alias):
            assert list(inspect.signature(getattr(mod, name)).parameters) == args


def test_torch_ops_are_registered():
    for name in REFERENCE_SIGNATURES:
        if name.endswith(("triton", "dejavu")):
            continue
        assert hasattr(torch.ops.flash_gemv, name)


def test_ops_reject_cpu_tensors():
    x = torch.randn(1, 1, 64)
    w = torch.randn(96, 64)
    with pytest.raises(RuntimeError, match="CUDA"):
        fg.flag_gemv_gemv_inner_fp32(x, w, w, w.t().contiguous(), 0.1)
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.flash_gemv.flag_gemv_gemv_inner_fp32(x, w, w, w.t().contiguous(), 0.1)
