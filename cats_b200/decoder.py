"""Greedy decode loop of a full Llama / Mistral decoder whose MLPs run the CATS kernels.

What the reference measures end to end (experiments/bench_sparse_inference_llama.py:51-101 and
the Mistral twin; timing of tokens 2..N with CUDA events in experiments/time_util_nofile.py:
2894-3004; caller shape inference.py:14-62) is HF ``generate`` over a model whose MLPs were
swapped by ``apply_sparse_silu_mlp``.  At B200 speeds a 7B token is ~2 ms of HBM time and an eager
HF step costs several times that in Python and launch overhead, so this module decodes straight
from the model's weight tensors:

* static KV cache ``[layers, B, kv_heads, max_len, head_dim]``, token ids, position and the
  attention mask all live on the device and are advanced by the step itself, so a step is a pure
  function of device state and the whole step is captured in a CUDA graph (one graph per bucket of
  256 cache positions, so attention does not read the unused tail of the cache);
* per layer: fused QKV projection, RoPE, cache write, SDPA, output projection (PyTorch / cuBLAS:
  not the path this library is about), then the MLP half in ONE launch of the library's kernel:
  ``cats_mlp`` with the fused tail ``resid += mlp(x); x_next = rmsnorm(resid) * w_next``, i.e.
  the residual add and the NEXT layer's input norm (the final norm after the last layer) come
  out of the MLP kernel;
* prefill runs the reference's rule for T > 1, the dense thresholded MLP
  (experiments/models/sparse_silu/ugly_utils.py:900-904);
* ``mlp="dense"`` runs the same loop with the plain SiLU-gated MLP (cuBLAS), the baseline;
  ``mlp="masked"`` the dense thresholded MLP in PyTorch (``sp_method = 0``), the parity reference.

Numerics follow HF's modelling code (RMS norm in fp32 then cast then weight; rotate-half RoPE from
the model's own ``inv_freq``; softmax scale ``head_dim ** -0.5``), checked against the HF forward
in the tests.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.nn.functional as F

from . import _lib, ops

BUCKET = 256


def _rmsnorm(h: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    hf = h.float()
    return w * (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)).to(h.dtype)


def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


class CatsDecoder:
    """Decode state and step function over the weights of an HF ``LlamaForCausalLM`` /
    ``MistralForCausalLM`` (or the Sparse* subclasses) that lives on one CUDA device.

    ``thresholds``: per-layer CATS thresholds; default: each layer's ``mlp.dead_threshold``.
    """

    def __init__(self, model, batch: int, max_len: int, mlp: str = "cats",
                 thresholds: Optional[List[float]] = None):
        if mlp not in ("cats", "dense", "masked"):
            raise RuntimeError(f"cats_b200.decoder: unknown mlp mode {mlp!r}")
        cfg = model.config
        self.model, self.mode = model, mlp
        self.B, self.max_len = batch, (max_len + BUCKET - 1) // BUCKET * BUCKET
        self.L = cfg.num_hidden_layers
        self.H, self.I = cfg.hidden_size, cfg.intermediate_size
        self.nh, self.nkv = cfg.num_attention_heads, cfg.num_key_value_heads
        self.hd = getattr(cfg, "head_dim", None) or self.H // self.nh
        self.eps = float(cfg.rms_norm_eps)
        emb = model.model.embed_tokens.weight
        self.dev, self.dt = emb.device, emb.dtype
        if self.dev.type != "cuda" and mlp == "cats":
            raise RuntimeError("cats_b200.decoder: the CATS MLP needs a CUDA device (no CPU path)")
        self.embed, self.lm_head = emb, model.lm_head.weight
        self.final_norm = model.model.norm.weight
        layers = model.model.layers
        self.wqkv = [torch.cat([l.self_attn.q_proj.weight, l.self_attn.k_proj.weight,
                                l.self_attn.v_proj.weight], 0).contiguous() for l in layers]
        self.wo = [l.self_attn.o_proj.weight for l in layers]
        self.ln1 = [l.input_layernorm.weight for l in layers]
        self.ln2 = [l.post_attention_layernorm.weight for l in layers]
        self.mlps = [l.mlp for l in layers]
        self.wg = [m.gate_proj.weight for m in self.mlps]
        self.wu = [m.up_proj.weight for m in self.mlps]
        self.wd = [m.down_proj.weight for m in self.mlps]
        self.thr = [float(t) for t in (thresholds if thresholds is not None else
                                       [getattr(m, "dead_threshold", 0.0) for m in self.mlps])]
        rot = model.model.rotary_emb
        pos = torch.arange(self.max_len, device=self.dev, dtype=torch.float32)
        freqs = torch.outer(pos, rot.inv_freq.to(self.dev).float())
        embd = torch.cat((freqs, freqs), -1)
        scale = float(getattr(rot, "attention_scaling", 1.0))
        self.cos, self.sin = (embd.cos() * scale).to(self.dt), (embd.sin() * scale).to(self.dt)

        z = lambda *s, dt=self.dt: torch.zeros(s, dtype=dt, device=self.dev)
        self.kc = z(self.L, batch, self.nkv, self.max_len, self.hd)
        self.vc = z(self.L, batch, self.nkv, self.max_len, self.hd)
        self.tok = z(batch, dt=torch.int64)
        self.pos = z(1, dt=torch.int64)                 # cache position of the token in self.tok
        self.h = z(batch, self.H)                       # residual stream of the current token
        self.x = z(batch, self.H)                       # normalised input of the next block
        self.x2 = z(batch, self.H)
        self.q = z(batch, self.nh, self.hd)
        self.logits = z(batch, cfg.vocab_size)          # logits of the latest step (static buffer)
        self.ar = torch.arange(self.max_len, device=self.dev)
        self.out_tokens: List[torch.Tensor] = []
        self.graphs = {}
        self.n_pos = 0                                  # host copy of self.pos
        if mlp == "cats":
            self.wdt = [m.packed_down() if hasattr(m, "packed_down") else ops.packed_wdt(m.down_proj.weight)
                        for m in self.mlps]
            self.ws = ops.Workspace(self.dev, self.H, self.I)
            self.code = ops.dtype_code(self.dt)
            self._fn = _lib.lib().cats_mlp
            for w in self.wg + self.wu + self.wdt:
                ops._req(w, "MLP weight", self.dt, self.dev)
        self.mlp_launches_per_step = self.L if mlp == "cats" else 0
        # batches: the density-aware switch to the dense tensor-core path (down_proj.weight is
        # at hand in its native layout)
        self.dense = (mlp == "cats" and ops.use_dense(batch, getattr(self.mlps[0], "sparsity_level", None))
                      and ops.dense_supported(batch, self.H, self.I, self.dt))
        if self.dense:
            self._fn_dense = _lib.lib().cats_mlp_dense

    # ---- pieces ---------------------------------------------------------------------------------
    def _attn_decode(self, l: int, x: torch.Tensor, bucket: int, cos, sin, mask) -> torch.Tensor:
        B, nh, nkv, hd = self.B, self.nh, self.nkv, self.hd
        qkv = F.linear(x, self.wqkv[l])
        if self.dev.type == "cuda":
            # RoPE + cache write in one launch (cats_rope_cache) instead of a dozen
            q = self.q
            ops.rope_cache(qkv, self.cos, self.sin, self.pos, q, self.kc[l], self.vc[l], nh, nkv)
        else:
            q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], -1)
            q, k = q.view(B, nh, hd), k.view(B, nkv, hd)
            q = q * cos + _rotate_half(q) * sin
            k = k * cos + _rotate_half(k) * sin
            self.kc[l].index_copy_(2, self.pos, k.unsqueeze(2))
            self.vc[l].index_copy_(2, self.pos, v.reshape(B, nkv, 1, hd))
        o = F.scaled_dot_product_attention(q.unsqueeze(2), self.kc[l][:, :, :bucket],
                                           self.vc[l][:, :, :bucket], attn_mask=mask,
                                           enable_gqa=nh != nkv)
        return F.linear(o.reshape(B, nh * hd), self.wo[l])

    def _next_norm_weight(self, l: int) -> torch.Tensor:
        return self.ln1[l + 1] if l + 1 < self.L else self.final_norm

    def _mlp_tail(self, l: int) -> None:
        """h += mlp(x2); x = rmsnorm(h) * (next block's norm weight)."""
        nw = self._next_norm_weight(l)
        if self.mode == "cats" and self.dense:
            st = self._fn_dense(self.x2.data_ptr(), self.wg[l].data_ptr(), self.wu[l].data_ptr(),
                                self.wd[l].data_ptr(), self.ws.ptr, self.ws.nbytes, self.B, self.H,
                                self.I, self.code, self.thr[l], None, _lib.OUT_STORE, self.h.data_ptr(),
                                self.x.data_ptr(), nw.data_ptr(), self.eps,
                                torch.cuda.current_stream(self.dev).cuda_stream)
            if st:
                _lib.check(st, "cats_mlp_dense")
            return
        if self.mode == "cats":
            st = self._fn(self.x2.data_ptr(), self.wg[l].data_ptr(), self.wu[l].data_ptr(),
                          self.wdt[l].data_ptr(), self.ws.ptr, self.ws.nbytes, self.B, self.H, self.I,
                          self.code, self.thr[l], None, _lib.OUT_STORE, self.h.data_ptr(),
                          self.x.data_ptr(), nw.data_ptr(), self.eps,
                          torch.cuda.current_stream(self.dev).cuda_stream)
            if st:
                _lib.check(st, "cats_mlp")
            return
        p = F.silu(F.linear(self.x2, self.wg[l]))
        if self.mode == "masked":
            p = torch.where(p.abs() <= self.thr[l], torch.zeros_like(p), p)
        y = F.linear(p * F.linear(self.x2, self.wu[l]), self.wd[l])
        if self.dev.type == "cuda":
            ops.tail(y, self.h, self.x, nw, self.eps)
        else:
            self.h.add_(y)
            self.x.copy_(_rmsnorm(self.h, nw, self.eps))

    @torch.no_grad()
    def _step(self, bucket: int) -> None:
        """One decode step on device state: consumes self.tok at self.pos, leaves the next token
        in self.tok and advances self.pos."""
        self.h.copy_(self.embed.index_select(0, self.tok))
        self.x.copy_(_rmsnorm(self.h, self.ln1[0], self.eps))
        # position-dependent pieces once per step, not once per layer
        cos, sin = self.cos.index_select(0, self.pos), self.sin.index_select(0, self.pos)  # [1, hd]
        mask = torch.where(self.ar[:bucket] <= self.pos, 0.0, float("-inf")).to(self.dt)
        mask = mask.view(1, 1, 1, bucket)
        for l in range(self.L):
            a = self._attn_decode(l, self.x, bucket, cos, sin, mask)
            if self.dev.type == "cuda":
                # h += attn; x2 = rmsnorm(h) * ln2 in one launch (cats_tail, the same kernel in
                # every mlp mode, so the comparison between the modes stays about the MLP)
                ops.tail(a, self.h, self.x2, self.ln2[l], self.eps)
            else:
                self.h.add_(a)
                self.x2.copy_(_rmsnorm(self.h, self.ln2[l], self.eps))
            self._mlp_tail(l)
        torch.matmul(self.x, self.lm_head.t(), out=self.logits)
        self.tok.copy_(self.logits.argmax(-1))
        self.pos.add_(1)

    # ---- prefill ----------------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Run the prompt (B, T) through the decoder, fill the cache and return the logits of its
        last position.  T > 1: the MLPs take the dense thresholded branch (dense in mode
        "dense"), as the reference's module does for prefill."""
        B, T = input_ids.shape
        assert B == self.B and T < self.max_len
        nh, nkv, hd = self.nh, self.nkv, self.hd
        h = self.embed[input_ids]                                     # [B, T, H]
        cos, sin = self.cos[:T].view(1, 1, T, hd), self.sin[:T].view(1, 1, T, hd)
        for l in range(self.L):
            x = _rmsnorm(h, self.ln1[l], self.eps)
            qkv = F.linear(x, self.wqkv[l])
            q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], -1)
            q = q.view(B, T, nh, hd).transpose(1, 2)
            k = k.view(B, T, nkv, hd).transpose(1, 2)
            v = v.view(B, T, nkv, hd).transpose(1, 2)
            q = q * cos + _rotate_half(q) * sin
            k = k * cos + _rotate_half(k) * sin
            self.kc[l][:, :, :T] = k
            self.vc[l][:, :, :T] = v
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=nh != nkv)
            h = h + F.linear(o.transpose(1, 2).reshape(B, T, nh * hd), self.wo[l])
            x2 = _rmsnorm(h, self.ln2[l], self.eps)
            p = F.silu(F.linear(x2, self.wg[l]))
            if self.mode != "dense":
                p = torch.where(p.abs() <= self.thr[l], torch.zeros_like(p), p)
            h = h + F.linear(p * F.linear(x2, self.wu[l]), self.wd[l])
        logits = F.linear(_rmsnorm(h[:, -1], self.final_norm, self.eps), self.lm_head)
        self.tok.copy_(logits.argmax(-1))
        self.pos.fill_(T)
        self.n_pos = T
        return logits

    # ---- decode -----------------------------------------------------------------------------------
    def _bucket(self, n_pos: int) -> int:
        return min(self.max_len, (n_pos + 1 + BUCKET - 1) // BUCKET * BUCKET)

    @torch.no_grad()
    def capture(self, first_pos: int, last_pos: int) -> None:
        """Record the decode step into CUDA graphs, one per cache bucket that positions
        first_pos..last_pos touch.  Runs two eager steps first (library warm-up) and restores the
        state they changed; capturing itself executes nothing."""
        keep = (self.tok.clone(), self.pos.clone(), self.h.clone(), self.x.clone())
        side = torch.cuda.Stream(self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):
            self.pos.fill_(min(first_pos, self.max_len - 3))
            for _ in range(2):
                self._step(self._bucket(first_pos))
        torch.cuda.current_stream(self.dev).wait_stream(side)
        torch.cuda.synchronize(self.dev)
        for b in sorted({self._bucket(p) for p in range(first_pos, last_pos + 1)}):
            if b in self.graphs:
                continue
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._step(b)
            self.graphs[b] = g
        self.tok.copy_(keep[0]); self.pos.copy_(keep[1]); self.h.copy_(keep[2]); self.x.copy_(keep[3])
        torch.cuda.synchronize(self.dev)

    @torch.no_grad()
    def decode(self, n_tokens: int, use_graph: bool = True, keep_logits: bool = False):
        """Generate ``n_tokens`` greedy tokens after ``prefill``.  Returns (tokens [B, n_tokens + 1]
        including the token the prefill produced, tokens/s of tokens 2..N timed with CUDA events
        on the device, list of logits if asked)."""
        stream = torch.cuda.current_stream(self.dev)
        toks, logs = [self.tok.clone()], []
        if self.n_pos + n_tokens >= self.max_len:
            raise RuntimeError("cats_b200.decoder: the KV cache is too short for this many tokens")
        if use_graph:
            self.capture(self.n_pos, self.n_pos + n_tokens - 1)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(n_tokens):
            b = self._bucket(self.n_pos)
            if use_graph:
                self.graphs[b].replay()
            else:
                self._step(b)
            self.n_pos += 1
            if i == 0:
                t0.record(stream)            # the reference's timer starts after the first token
            toks.append(self.tok.clone())
            if keep_logits:
                logs.append(self.logits.clone())
        t1.record(stream)
        t1.synchronize()
        dt_ms = t0.elapsed_time(t1)
        tps = (n_tokens - 1) * self.B / (dt_ms * 1e-3) if n_tokens > 1 and dt_ms > 0 else float("nan")
        return torch.stack(toks, 1), tps, logs


# ---- model construction (random init: there are no checkpoints offline) ---------------------------
def build_random_model(family: str, dtype=torch.float16, device="cuda", layers: Optional[int] = None,
                       seed: int = 0, **overrides):
    """HF Llama-2-7B / Mistral-7B architecture with random N(0, 0.02^2) weights, MLPs swapped for
    the CATS module (``apply_sparse_silu_mlp``), built on ``device`` in ``dtype``."""
    from transformers import LlamaConfig, MistralConfig

    from . import sparse_silu as S

    if family == "llama":
        cfg = LlamaConfig(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                          num_attention_heads=32, num_key_value_heads=32, vocab_size=32000,
                          max_position_embeddings=4096, rms_norm_eps=1e-5, initializer_range=0.02)
        cls, mt = S.SparseLlamaForCausalLM, S.LLAMA
    elif family == "mistral":
        cfg = MistralConfig(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                            num_attention_heads=32, num_key_value_heads=8, vocab_size=32000,
                            max_position_embeddings=8192, rms_norm_eps=1e-5, initializer_range=0.02,
                            sliding_window=None)
        cls, mt = S.SparseMistralforCausalLM, S.MISTRAL
    else:
        raise RuntimeError(f"cats_b200.decoder: unknown family {family!r}")
    if layers is not None:
        cfg.num_hidden_layers = layers
    for k, v in overrides.items():
        setattr(cfg, k, v)
    cfg = S.get_sparse_config(cfg, model_type=mt, use_sparse_model=True)
    cfg.use_relu = False
    torch.manual_seed(seed)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with torch.device(device):
            model = cls(cfg)
    finally:
        torch.set_default_dtype(prev)
    model.eval()
    S.enable_sparse_silu(model)
    return model


@torch.no_grad()
def calibrate(model, sparsity: float, n_prompts: int = 4, prompt_len: int = 128, seed: int = 1):
    """Per-layer thresholds the reference's way: ``activate_stats`` -> forward passes over
    calibration prompts (uniform-random token ids here) with the activation histograms collected
    on the device -> ``set_sparse_threshold(model, sparsity)`` -> ``deactivate_stats``.
    Returns the list of thresholds."""
    from . import sparse_silu as S

    dev = model.model.embed_tokens.weight.device
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    S.disable_sparse_silu(model)          # histograms of the un-thresholded activations ...
    for l in model.model.layers:
        l.mlp.kill_sparse_swish_outputs = True   # ... but the statistics branch is the sparse one
        l.mlp.dead_threshold = 0.0
    S.activate_stats(model)
    for _ in range(n_prompts):
        ids = torch.randint(0, model.config.vocab_size, (1, prompt_len), generator=g).to(dev)
        model(ids, use_cache=False)
    S.set_sparse_threshold(model, sparsity)
    S.deactivate_stats(model)
    return [float(l.mlp.dead_threshold) for l in model.model.layers]
