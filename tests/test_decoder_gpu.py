"""Full-decoder decode on the GPU: the CATS kernels inside a random-init Llama / Mistral decoder
against the same decoder with the dense thresholded PyTorch MLP (the reference's ``sp_method = 0``
branch), 16 greedy tokens, eager and replayed from CUDA graphs; and HF ``generate`` over the
swapped-in modules (the reference's own call path)."""
import numpy as np
import pytest
import torch

from oracle import cats_oracle as O

pytestmark = pytest.mark.gpu

SMALL = dict(hidden_size=1024, intermediate_size=2752, num_attention_heads=8, vocab_size=2000,
             head_dim=128)


def to_np(t):
    return t.detach().float().cpu().numpy()


def small_model(family, layers, dev):
    from cats_b200 import decoder as D

    kv = 8 if family == "llama" else 2
    model = D.build_random_model(family, torch.float16, dev, layers=layers, seed=3,
                                 num_key_value_heads=kv, **SMALL)
    thr = D.calibrate(model, 0.5, n_prompts=2, prompt_len=64)
    return model, thr


@pytest.mark.parametrize("family,B", [("llama", 1), ("mistral", 4), ("mistral", 8)])
def test_cats_decoder_matches_the_dense_thresholded_decoder(family, B, cuda_device):
    from cats_b200 import decoder as D

    model, thr = small_model(family, 3, cuda_device)
    assert all(t > 0 for t in thr), thr
    ids = torch.randint(0, SMALL["vocab_size"], (B, 40), device=cuda_device)
    ref = D.CatsDecoder(model, B, 400, mlp="masked", thresholds=thr)
    cats = D.CatsDecoder(model, B, 400, mlp="cats", thresholds=thr)
    l0 = ref.prefill(ids)
    l1 = cats.prefill(ids)
    assert O.rel_l2(to_np(l1), to_np(l0)) <= 1e-3          # same PyTorch prefill
    errs = []
    for step in range(16):
        cats.tok.copy_(ref.tok)                             # teacher forcing: same token sequence
        ref._step(D.BUCKET)
        cats._step(D.BUCKET)
        errs.append(O.rel_l2(to_np(cats.logits), to_np(ref.logits)))
    torch.cuda.synchronize()
    assert cats.ws.counters()[1] == 0
    # one mask flip next to the threshold moves a 2752-neuron layer's output by a percent or two
    # (the reference path rounds the gate values to fp16 before it compares them)
    assert float(np.median(errs)) <= 3e-2 and max(errs) <= 8e-2, errs


def test_graph_replay_equals_eager(cuda_device):
    from cats_b200 import decoder as D

    model, thr = small_model("llama", 2, cuda_device)
    ids = torch.randint(0, SMALL["vocab_size"], (1, 250), device=cuda_device)
    runs = []
    for use_graph in (False, True):
        dec = D.CatsDecoder(model, 1, 300, mlp="cats", thresholds=thr)
        dec.prefill(ids)
        toks, tps, logs = dec.decode(12, use_graph=use_graph, keep_logits=True)   # crosses a bucket
        runs.append((toks, torch.stack(logs)))
        assert tps > 0
        if use_graph:
            assert len(dec.graphs) == 2
    # same kernels, same order of operations: the logits agree to rounding; tokens may only differ
    # where two logits tie within that rounding
    assert O.rel_l2(to_np(runs[1][1][:4]), to_np(runs[0][1][:4])) <= 2e-2
    assert torch.equal(runs[0][0][:, :2], runs[1][0][:, :2])


def test_hf_generate_runs_the_cuda_path_through_the_swapped_modules(cuda_device):
    """The reference's call path: ``model.generate`` over modules with ``is_profile`` set
    (bench_sparse_inference_llama.py:66-98).  Decode steps reach ``CatsSparseSiluMLP.forward`` with
    one token and take the CUDA path; the result must follow the ``sp_method = 0`` run."""
    model, thr = small_model("llama", 2, cuda_device)
    ids = torch.randint(0, SMALL["vocab_size"], (1, 16), device=cuda_device)
    outs = {}
    calls = {"n": 0}
    mlp0 = model.model.layers[0].mlp
    orig = mlp0._cuda_decode

    def counted(x):
        calls["n"] += 1
        return orig(x)

    mlp0._cuda_decode = counted
    for method in (0, 2):
        for m in model.model.layers:
            m.mlp.is_profile = True
            m.mlp.sp_method = method
            if method == 2:
                m.mlp.wdown_t = m.mlp.down_proj.weight.t().contiguous()
        with torch.no_grad():
            out = model.generate(input_ids=ids, max_length=16 + 6, use_cache=True, do_sample=False,
                                 pad_token_id=0, output_logits=True, return_dict_in_generate=True)
        outs[method] = out
    assert calls["n"] >= 5                                   # every decode step after the prefill
    la, lb = torch.stack(outs[0].logits), torch.stack(outs[2].logits)
    assert O.rel_l2(to_np(lb[:2]), to_np(la[:2])) <= 3e-2   # first steps: same token history


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv", [(8, 8), (8, 2)])
def test_rope_and_cache_write_equal_the_elementwise_launches(dt, nh, nkv, cuda_device):
    from cats_b200 import ops
    from cats_b200.decoder import _rotate_half

    B, hd, max_len = 3, 128, 64
    dev = cuda_device
    torch.manual_seed(1)
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, device=dev).to(dt)
    ang = torch.outer(torch.arange(max_len, device=dev).float(), torch.rand(hd // 2, device=dev))
    emb = torch.cat((ang, ang), -1)
    cos, sin = emb.cos().to(dt), emb.sin().to(dt)
    for p in (0, 17, max_len - 1):
        pos = torch.tensor([p], device=dev)
        kc = torch.zeros(B, nkv, max_len, hd, device=dev, dtype=dt)
        vc = torch.zeros_like(kc)
        q_out = torch.empty(B, nh, hd, device=dev, dtype=dt)
        ops.rope_cache(qkv, cos, sin, pos, q_out, kc, vc, nh, nkv)
        q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], -1)
        q, k = q.view(B, nh, hd), k.view(B, nkv, hd)
        c, s = cos[p:p + 1], sin[p:p + 1]
        assert torch.equal(q_out, q * c + _rotate_half(q) * s)
        assert torch.equal(kc[:, :, p], k * c + _rotate_half(k) * s)
        assert torch.equal(vc[:, :, p], v.reshape(B, nkv, hd))
        kc[:, :, p] = 0
        vc[:, :, p] = 0
        assert float(kc.abs().max()) == 0 and float(vc.abs().max()) == 0     # nothing else written
