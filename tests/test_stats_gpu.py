"""Device-side activation statistics (cats_histogram, cats_histogram_threshold) against the
reference's collect_stats / get_threshold: integer counts bit-exact, thresholds equal."""
import numpy as np
import pytest
import torch

from conftest import golden_names, load_golden
from oracle import cats_oracle as O

pytestmark = pytest.mark.gpu


def dev_bins(device):
    return torch.from_numpy(O.reference_bins()).to(device, torch.float32)


def test_histograms_equal_the_reference_collect_stats_golden(cuda_device):
    from cats_b200 import ops

    g = load_golden("get_threshold_0")
    edges = dev_bins(cuda_device)
    pre = torch.from_numpy(g["pre"]).to(cuda_device)
    post = torch.from_numpy(g["post"]).to(cuda_device)
    pre_counts = ops.histogram(pre, edges)
    post_counts = ops.histogram(post, edges, take_abs=True)
    assert np.array_equal(pre_counts.cpu().numpy(), g["pre_counts"].astype(np.int64))
    assert np.array_equal(post_counts.cpu().numpy(), g["counts"].astype(np.int64))


@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n,offset", [(1, 0), (7, 3), (4099, 1), (512 * 14336 + 5, 0)])
def test_histogram_matches_torch_histogram(dt, n, offset, cuda_device):
    from cats_b200 import ops

    gen = torch.Generator().manual_seed(n + offset)
    base = (torch.randn(n + offset, generator=gen) * 1.3).to(dt)
    edges_cpu = torch.from_numpy(O.reference_bins())
    # values exactly on edges, at the ends, infinities and a NaN
    special = torch.tensor([-1.0, 1.0, 0.0, float(edges_cpu[500]), float(edges_cpu[501]),
                            float("inf"), float("-inf"), float("nan"), 3.5, -7.0]).to(dt)
    k = min(special.numel(), n)
    base[offset:offset + k] = special[:k]
    v = base.to(cuda_device)[offset:]              # offset: not 16-byte aligned
    edges = edges_cpu.to(cuda_device)
    counts = ops.histogram(v, edges)
    counts = ops.histogram(v, edges, counts, take_abs=True)     # accumulates
    ref_pre, ref_post = O.activation_histograms(base[offset:].float().numpy(),
                                                base[offset:].float().numpy(), edges_cpu.numpy())
    assert np.array_equal(counts.cpu().numpy(), ref_pre + ref_post)
    finite = int(torch.isnan(base[offset:].float()).logical_not().sum())
    assert int(counts.sum()) == 2 * finite


def test_histogram_with_few_uneven_edges(cuda_device):
    from cats_b200 import ops

    edges_cpu = torch.tensor([-2.0, -0.5, -0.25, 0.0, 0.125, 4.0])
    v_cpu = torch.tensor([-3.0, -2.0, -0.5, -0.3, 0.0, 0.1, 0.125, 3.9, 4.0, 4.1, -0.25])
    counts = ops.histogram(v_cpu.to(cuda_device), edges_cpu.to(cuda_device))
    ref = torch.histogram(v_cpu, bins=edges_cpu)[0].to(torch.int64)
    assert torch.equal(counts.cpu(), ref)


@pytest.mark.parametrize("name", golden_names("get_threshold_"))
def test_threshold_equals_the_reference_get_threshold_golden(name, cuda_device):
    from cats_b200 import ops

    g = load_golden(name)
    counts = torch.from_numpy(g["counts"].astype(np.int64)).to(cuda_device)
    t = ops.histogram_threshold(counts, dev_bins(cuda_device), float(g["sparsity"]))
    assert float(t.item()) == float(np.float32(g["threshold"]))


def test_threshold_on_random_histograms_matches_the_oracle(cuda_device):
    from cats_b200 import ops

    rng = np.random.default_rng(3)
    edges = dev_bins(cuda_device)
    for trial in range(20):
        counts = rng.integers(0, 4000, size=999).astype(np.int64)
        counts[rng.integers(0, 999, size=300)] = 0
        for s in (0.0, 0.1, 0.5, 0.9, 0.999, 1.0):
            t = ops.histogram_threshold(torch.from_numpy(counts).to(cuda_device), edges, s)
            ref = O.get_threshold(O.reference_bins(), counts.astype(np.float32), s)
            assert float(t.item()) == float(ref), (trial, s)


def test_module_collects_cuda_activations_on_the_device(cuda_device):
    from cats_b200 import sparse_silu as S

    cfg = {"hidden_size": 64, "intermediate_size": 96}
    mlp = S.LlamaSparseSiluMLP(cfg).to(cuda_device)
    mlp.activate_stats()
    g = load_golden("get_threshold_0")
    pre = torch.from_numpy(g["pre"]).to(cuda_device)
    post = torch.from_numpy(g["post"]).to(cuda_device)
    mlp.collect_stats(pre, post)
    mlp.collect_stats(pre.cpu(), post.cpu())          # the host path still adds to the same totals
    assert torch.equal(mlp.pre_act_hist_counts, torch.from_numpy(2 * g["pre_counts"]).float())
    assert torch.equal(mlp.post_act_hist_counts, torch.from_numpy(2 * g["counts"]).float())
    thr = S.get_threshold(mlp.histogram_bins, mlp.post_act_hist_counts.clone(), float(g["sparsity"]))
    assert float(thr) == float(np.float32(g["threshold"]))
