"""The CPU oracle against the golden vectors produced by the reference's own module."""
import numpy as np
import pytest

from conftest import MLP_GOLDEN, golden_names, load_golden
from oracle import cats_oracle as O

# tolerance of the oracle (fp32 numpy) against the reference's torch output per storage dtype:
# 16-bit cases differ by the reference's rounding of every intermediate to 16 bits.
TOL = {"float32": 2e-6, "float16": 4e-3, "bfloat16": 3e-2}


@pytest.mark.parametrize("name", MLP_GOLDEN)
def test_dense_masked_mlp_matches_reference(name):
    g = load_golden(name)
    dt = str(g["dtype"])
    res = O.dense_masked_mlp(g["x"], g["wg"], g["wu"], g["wd"], float(g["threshold"]))
    assert res["out"].shape == g["y"].shape
    if dt == "float32":
        # same mask as the reference (its post-activation is stored in the file)
        ref_mask = np.abs(g["post_act"]) > np.float32(g["threshold"])
        flips, outside = O.mask_band_check(g["post_act"], res["mask"], float(g["threshold"]))
        assert outside == 0
        if flips == 0:
            assert np.array_equal(res["mask"], ref_mask)
            assert O.rel_l2(res["out"], g["y"]) < TOL[dt]
    else:
        # the 16-bit reference thresholds a rounded activation: compare with its own mask
        ref_mask = np.abs(g["post_act"]) > np.float32(g["threshold"])
        res = O.dense_masked_mlp(g["x"], g["wg"], g["wu"], g["wd"], float(g["threshold"]),
                                 mask=ref_mask)
        assert O.rel_l2(res["out"], g["y"]) < TOL[dt]


@pytest.mark.parametrize("name", [n for n in MLP_GOLDEN if "f32" in n])
def test_non_profile_kill_path_is_the_same_function(name):
    g = load_golden(name)
    assert np.array_equal(g["y"], g["y_kill"])


@pytest.mark.parametrize("name", [n for n in MLP_GOLDEN if "f32" in n])
def test_fp64_oracle_agrees_with_fp32(name):
    g = load_golden(name)
    a = O.dense_masked_mlp(g["x"], g["wg"], g["wu"], g["wd"], float(g["threshold"]))
    b = O.dense_masked_mlp(g["x"], g["wg"], g["wu"], g["wd"], float(g["threshold"]),
                           dtype=np.float64)
    flips, outside = O.mask_band_check(b["post_act"], a["mask"], float(g["threshold"]))
    assert outside == 0
    if flips == 0:
        assert O.rel_l2(a["out"], b["out"]) < 1e-5


@pytest.mark.parametrize("name", [n for n in MLP_GOLDEN if "f32" in n])
def test_test_file_golden_formula(name):
    g = load_golden(name)
    y = O.test_file_golden(g["x"], g["wg"].T, g["wu"].T, g["wd"].T, float(g["threshold"]))
    assert O.rel_l2(y, g["y"]) < 2e-6


@pytest.mark.parametrize("name", [n for n in MLP_GOLDEN if "f32" in n])
def test_sp_mask_branch(name):
    g = load_golden(name)
    thr = float(g["threshold"])
    x, wg, wu, wd = (g[k].astype(np.float32) for k in ("x", "wg", "wu", "wd"))
    pre = (x @ wg.T) * g["sp_mask"]
    y = (O.sparse_silu(pre, np.float32(thr)) * (x @ wu.T)) @ wd.T
    assert O.rel_l2(y, g["y_spmask"]) < 2e-6


@pytest.mark.parametrize("name", golden_names("sparse_silu_"))
def test_sparse_silu(name):
    g = load_golden(name)
    y = O.sparse_silu(g["a"].astype(np.float32), np.float32(g["threshold"]))
    assert np.allclose(y, g["y"], rtol=1e-6, atol=1e-7)
    # for t >= 0 SparseSiLU is "keep where |act| > t" — the rule the kernels implement
    act = O.silu(g["a"].astype(np.float32))
    assert np.array_equal(y != 0, (np.abs(act) > np.float32(g["threshold"])) & (act != 0))


@pytest.mark.parametrize("name", golden_names("get_threshold_"))
def test_get_threshold(name):
    g = load_golden(name)
    t = O.get_threshold(g["bins"], g["counts"], float(g["sparsity"]))
    assert float(t) == pytest.approx(float(g["threshold"]), abs=0)


def test_union_mask_rule():
    m = np.array([[1, 0, 0, 1], [0, 0, 1, 1]], dtype=bool)
    assert O.union_mask(m).tolist() == [True, False, True, True]


def test_quantile_threshold_hits_sparsity():
    rng = np.random.default_rng(0)
    wg = rng.normal(0, 0.02, (512, 256)).astype(np.float32)
    xc = rng.normal(0, 1, (256, 256)).astype(np.float32)
    xc /= np.sqrt((xc ** 2).mean(-1, keepdims=True))
    for s in (0.3, 0.5, 0.9):
        t = O.quantile_threshold(xc, wg, s)
        p = np.abs(O.silu(xc @ wg.T))
        assert abs((p <= t).mean() - s) <= 1.0 / p.size + 1e-12


def test_mlp_stack_is_chain_of_layers():
    rng = np.random.default_rng(1)
    H, I = 64, 96
    layers = [tuple(rng.normal(0, 0.2, s).astype(np.float32) for s in ((I, H), (I, H), (H, I)))
              for _ in range(3)]
    x0 = rng.normal(0, 1, (1, H)).astype(np.float32)
    x, r, counts = O.mlp_stack(x0, layers, [0.1, 0.1, 0.1])
    xr, rr = x0.copy(), x0.copy()
    for wg, wu, wd in layers:
        rr = rr + O.dense_masked_mlp(xr, wg, wu, wd, 0.1)["out"]
        xr = O.rmsnorm(rr)
    assert np.allclose(x, xr) and np.allclose(r, rr) and len(counts) == 3


def test_activation_histograms_match_the_reference_collect_stats():
    """The oracle's histograms against the counts the reference's own collect_stats produced."""
    g = load_golden("get_threshold_0")
    pre, post = O.activation_histograms(g["pre"], g["post"], g["bins"])
    assert np.array_equal(pre, g["pre_counts"].astype(np.int64))
    assert np.array_equal(post, g["counts"].astype(np.int64))
    assert np.array_equal(O.reference_bins().astype(np.float64), g["bins"])
