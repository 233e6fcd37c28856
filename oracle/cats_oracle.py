"""CPU oracle for the CATS thresholded sparse-MLP decode path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product (``cats_b200/``, ``flash_gemv/``) imports this file.  It is used by
``tests/``, by ``__graft_entry__.smoke()`` and by ``bench.py``'s CPU-baseline / reference arm as
the checker and as the timed CPU restatement of the reference — never as the thing shipped.

What it restates (reference = ScalingIntelligence/CATS):
  * the dense thresholded MLP, experiments/models/sparse_silu/ugly_utils.py:896-899 (identical
    at :901-904 for prefill and :557-566 in the Mistral class) — ``dense_masked_mlp`` (numpy,
    any float width) and ``torch_dense_masked_mlp`` (the same four torch calls the reference
    makes, used for CPU timing);
  * the golden formula of the reference's kernel test, flash_gemv/test/test_fuse_gemv_cmp.py:459-462
    (same arithmetic written with matmuls on (H, I)-layout weights) — ``test_file_golden``;
  * ``SparseSiLU``, ugly_utils.py:80-92 — ``sparse_silu``;
  * the batch rule: every token has its own mask; a weight row is *loaded* when any token needs it
    (flash_gemv/csrc/cuda/fuse_gemv_cmp_cuda.cu:1488-1495, 1542-1548) — ``union_mask``;
  * ``get_threshold``, ugly_utils.py:236-245 — histogram CDF + searchsorted(side="right").

Parity is PINNED: ``tests/golden/*.npz`` were produced by importing the reference's own module
(with its missing plotting / training imports stubbed out) and running its ``forward``; see
``tests/golden/make_golden.py``.  ``tests/test_oracle_golden.py`` checks every function here
against those files.

Arithmetic of the third-party library the reference relies on: the dense path is PyTorch's
``F.linear`` / ``F.silu`` (reference pins torch 1.13.1, all-pkgs.txt:304; the golden files were made
with the torch of this image).  SiLU(a) = a / (1 + exp(-a)); linear = plain inner products.
"""
from __future__ import annotations

import numpy as np


def silu(a: np.ndarray) -> np.ndarray:
    """SiLU in the array's own float width."""
    a = np.asarray(a)
    with np.errstate(over="ignore"):
        return a / (1 + np.exp(-a))


def dense_masked_mlp(x, wg, wu, wd, threshold, dtype=np.float32, mask=None):
    """The reference's dense thresholded MLP (ugly_utils.py:896-899).

    x (..., H); wg, wu (I, H); wd (H, I) — nn.Linear layouts.  ``dtype`` is the arithmetic width
    (float32 = "the fp32 reference" of the parity tolerance, float64 = tie-breaker).
    ``mask`` (..., I) bool overrides the threshold decision (used to compare outputs when a
    kernel's mask differs inside the allowed band around the threshold).
    Returns a dict: out (..., H), post_act (..., I) before masking, mask (..., I) bool (active
    neurons: |post_act| > threshold), inter (..., I) = masked post_act * up.
    """
    x = np.asarray(x, dtype=dtype)
    wg = np.asarray(wg, dtype=dtype)
    wu = np.asarray(wu, dtype=dtype)
    wd = np.asarray(wd, dtype=dtype)
    post_act = silu(x @ wg.T)
    if mask is None:
        dead = np.abs(post_act) <= dtype(threshold)
        mask = ~dead
    masked = np.where(mask, post_act, dtype(0))
    inter = masked * (x @ wu.T)
    out = inter @ wd.T
    return {"out": out, "post_act": post_act, "mask": mask, "inter": inter}


def test_file_golden(x, wgate_hi, wup_hi, wdown_ih, threshold, dtype=np.float32):
    """Golden of flash_gemv/test/test_fuse_gemv_cmp.py:459-462: weights given as (H, I), (H, I),
    (I, H) and used as right-hand matmul operands."""
    x = np.asarray(x, dtype=dtype)
    gv = silu(x @ np.asarray(wgate_hi, dtype=dtype))
    gu = (x @ np.asarray(wup_hi, dtype=dtype)) * gv
    gu = np.where(np.abs(gv) <= dtype(threshold), dtype(0), gu)
    return gu @ np.asarray(wdown_ih, dtype=dtype)


test_file_golden.__test__ = False  # not a pytest test despite its name


def sparse_silu(a, threshold):
    """SparseSiLU (ugly_utils.py:80-92): Threshold(t, 0)(act) - Threshold(t, 0)(-act), i.e. act
    where act > t, act where -act > t, else 0."""
    act = silu(np.asarray(a))
    pos = np.where(act > threshold, act, 0)
    neg = np.where(-act > threshold, -act, 0)
    return pos - neg


def union_mask(mask: np.ndarray) -> np.ndarray:
    """Rows that must be loaded for a batch: active for any token (mask (B, I) -> (I,))."""
    mask = np.asarray(mask, dtype=bool)
    return mask.reshape(-1, mask.shape[-1]).any(axis=0)


def get_threshold(bin_edges, histogram_counts, sparsity_level):
    """ugly_utils.py:236-245: normalise, cumsum, searchsorted(side='right'), take that edge —
    with the reference's own torch calls on float32 tensors (torch's CPU cumsum keeps its running
    sum in double and rounds every element to float32; a float32 running sum can land one bin
    away when the CDF passes within an ulp of the sparsity level)."""
    import torch

    counts = torch.as_tensor(np.asarray(histogram_counts, dtype=np.float32)).clone()
    counts /= counts.sum()
    idx = int(torch.searchsorted(counts.cumsum(0), float(sparsity_level), side="right"))
    return np.asarray(bin_edges)[idx]


def quantile_threshold(x_calib, wg, sparsity, dtype=np.float32):
    """Threshold used by the synthetic benchmark configurations: the ``sparsity`` quantile of
    |SiLU(Wg x)| pooled over all calibration vectors and neurons (k-th smallest value, so that
    exactly floor(sparsity * count) pooled values are <= t... up to ties)."""
    p = np.abs(silu(np.asarray(x_calib, dtype=dtype) @ np.asarray(wg, dtype=dtype).T)).ravel()
    k = int(sparsity * p.size)
    if k <= 0:
        return float(-1.0)
    return float(np.partition(p, k - 1)[k - 1])


def rmsnorm(r, eps=1e-6, weight=None, dtype=np.float32):
    r = np.asarray(r, dtype=dtype)
    y = r / np.sqrt(np.mean(r * r, axis=-1, keepdims=True) + dtype(eps))
    return y if weight is None else y * np.asarray(weight, dtype=dtype)


def mlp_stack(x0, layers, thresholds, eps=1e-6, dtype=np.float32, round_to=None):
    """Chain of CATS MLPs with a residual stream and RMS norm between layers, as the decoder
    does around its MLP halves (ugly_utils.py:1036-1057 restated for the MLP only):
        r_0 = x_0;  y_l = mlp_l(x_l);  r_{l+1} = r_l + y_l;  x_{l+1} = r_{l+1} / rms(r_{l+1})
    ``layers`` = [(wg, wu, wd_HI), ...].  ``round_to`` (np.float16 or a callable) models the
    storage type of r and x between layers.  Returns (x_L, r_L, [n_active per layer])."""
    def rnd(a):
        if round_to is None:
            return a
        if callable(round_to) and not isinstance(round_to, type):
            return round_to(a)
        return np.asarray(a).astype(round_to).astype(dtype)

    x = np.asarray(x0, dtype=dtype)
    r = x.copy()
    counts = []
    for (wg, wu, wd), t in zip(layers, thresholds):
        res = dense_masked_mlp(x, wg, wu, wd, t, dtype=dtype)
        counts.append(int(union_mask(res["mask"]).sum()))
        r = rnd(r + res["out"])
        x = rnd(rmsnorm(r, eps, dtype=dtype))
    return x, r, counts


def mask_band_check(post_act_ref, mask_kernel, threshold, rel=1e-3):
    """Compare a kernel's mask with the oracle's.  Returns (n_flips, n_outside): flips are
    positions where the masks differ; ``n_outside`` counts flips whose reference gate value is
    NOT within ``rel`` (relative) of the threshold — the parity bar requires n_outside == 0."""
    post = np.abs(np.asarray(post_act_ref, dtype=np.float64))
    ref_mask = post > float(threshold)
    flips = ref_mask != np.asarray(mask_kernel, dtype=bool)
    band = np.abs(post - float(threshold)) <= rel * abs(float(threshold))
    return int(flips.sum()), int((flips & ~band).sum())


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / den) if den > 0 else float(np.linalg.norm(a - b))


# --------------------------------------------------------------------------------------------
# torch restatement (same calls as the reference) — CPU timing and cross-checks
# --------------------------------------------------------------------------------------------
def torch_dense_masked_mlp(x, wg, wu, wd, threshold):
    """ugly_utils.py:896-899 with the module's nn.Linear / SiLU calls written functionally."""
    import torch
    import torch.nn.functional as F

    post_act = F.silu(F.linear(x, wg))
    dead_neurons = post_act.abs() <= threshold
    post_act[dead_neurons] = 0
    return F.linear(post_act * F.linear(x, wu), wd)


def activation_histograms(pre_activation, post_activation, bins):
    """The two histograms of collect_stats (ugly_utils.py:514-522): torch.histogram of the
    pre-activations and of |post-activations| over ``bins`` (float32 edges).  Returns int64
    numpy arrays (pre_counts, post_counts)."""
    import torch

    pre = torch.as_tensor(np.asarray(pre_activation, dtype=np.float32)).flatten()
    post = torch.as_tensor(np.asarray(post_activation, dtype=np.float32)).flatten()
    edges = torch.as_tensor(np.asarray(bins, dtype=np.float32))
    return (torch.histogram(pre, bins=edges)[0].numpy().astype(np.int64),
            torch.histogram(torch.abs(post), bins=edges)[0].numpy().astype(np.int64))


def reference_bins(num_bins=1000):
    """-inf, 998 points on [-1, 1], +inf (ugly_utils.py:491-493)."""
    import torch

    b = torch.linspace(-1, 1, num_bins - 2)
    return torch.cat([torch.tensor([-torch.inf]), b, torch.tensor([torch.inf])]).numpy()
