"""The dense tensor-core path (cats_mlp_dense: TMA + tcgen05.mma + tensor memory) against the CPU
oracle: per-token masks, every batch size up to 16, the model shapes, the fused tail."""
import numpy as np
import pytest
import torch

from oracle import cats_oracle as O

pytestmark = pytest.mark.gpu


def to_np(t):
    return t.detach().float().cpu().numpy()


def case(H, I, B, dt, sparsity, seed, dev):
    from cats_b200 import synth

    layer = synth.make_layer(H, I, dt, dev, seed, sparsity=sparsity,
                             std=0.02 if H >= 1024 else 1.3 / np.sqrt(H))
    x = synth.make_x(B, H, dt, dev, seed + 77)
    return x, layer, layer.wdt.t().contiguous()


def check(x, layer, wd, B, H, I, what):
    """out against the oracle (with the kernel's own mask where a gate value sits within the
    1e-3 band of the threshold; the mask itself is taken from stage 1 of the sparse path, which
    test_parity_gpu holds to the band rule) and the union count against the mask."""
    from cats_b200 import ops

    out = ops.mlp_dense(x, layer.wg, layer.wu, wd, layer.threshold)
    ws = ops.get_workspace(x.device, H, I)
    n_active, status = ws.counters()
    assert out.shape == x.shape and status == 0
    xn = to_np(x).reshape(B, H)
    ref64 = O.dense_masked_mlp(xn, to_np(layer.wg), to_np(layer.wu), to_np(wd), layer.threshold,
                               dtype=np.float64)
    union = int(O.union_mask(ref64["mask"]).sum())
    band = int((np.abs(np.abs(ref64["post_act"]) - layer.threshold) <= 1e-3 * layer.threshold).sum())
    assert abs(n_active - union) <= band, (what, n_active, union, band)
    ref32 = O.dense_masked_mlp(xn, to_np(layer.wg), to_np(layer.wu), to_np(wd), layer.threshold)
    err = O.rel_l2(to_np(out).reshape(B, H), ref32["out"])
    # gate * up is rounded to the storage type between the GEMMs and a gate value inside the band
    # may fall on the other side: 1e-2 is the bar for 16-bit runs
    assert err <= 1e-2, (what, err)
    return out


@pytest.mark.parametrize("B", [1, 2, 3, 4, 5, 8, 13, 16])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_batches_at_a_small_shape(B, dt, cuda_device):
    from cats_b200 import ops

    H, I = 1024, 2752
    assert ops.dense_supported(B, H, I, dt)
    x, layer, wd = case(H, I, B, dt, 0.7, 11 + B, cuda_device)
    check(x, layer, wd, B, H, I, f"B={B}")


@pytest.mark.parametrize("H,I,B,dt,sparsity", [
    (4096, 14336, 8, torch.float16, 0.5),
    (4096, 14336, 16, torch.bfloat16, 0.5),
    (4096, 14336, 4, torch.float16, 0.9),
    (4096, 11008, 2, torch.float16, 0.5),
    (8192, 28672, 8, torch.bfloat16, 0.7),      # two row tiles per CTA
    (128, 64, 3, torch.float16, 0.5),           # smallest supported shape: most CTAs idle
    (256, 4096, 16, torch.bfloat16, 0.3),
])
def test_model_and_odd_shapes(H, I, B, dt, sparsity, cuda_device):
    x, layer, wd = case(H, I, B, dt, sparsity, 5, cuda_device)
    check(x, layer, wd, B, H, I, f"{H}x{I} B={B}")


def test_empty_and_full_active_sets(cuda_device):
    from cats_b200 import ops

    H, I, B = 1024, 2752, 4
    x, layer, wd = case(H, I, B, torch.float16, 0.5, 9, cuda_device)
    out = ops.mlp_dense(x, layer.wg, layer.wu, wd, 1e9)            # nothing active
    assert float(out.abs().max()) == 0.0
    assert ops.get_workspace(cuda_device, H, I).counters()[0] == 0
    out = ops.mlp_dense(x, layer.wg, layer.wu, wd, -1.0)           # everything active
    ref = O.dense_masked_mlp(to_np(x).reshape(B, H), to_np(layer.wg), to_np(layer.wu), to_np(wd), -1.0)
    assert O.rel_l2(to_np(out).reshape(B, H), ref["out"]) <= 1e-2
    assert ops.get_workspace(cuda_device, H, I).counters()[0] == I


def test_fused_tail_and_repeated_calls_on_one_workspace(cuda_device):
    from cats_b200 import ops

    H, I, B, dt = 1024, 2752, 8, torch.bfloat16
    x, layer, wd = case(H, I, B, dt, 0.5, 51, cuda_device)
    plain = ops.mlp_dense(x, layer.wg, layer.wu, wd, layer.threshold).reshape(B, H)
    for rep in range(3):
        resid = torch.randn((B, H), device=cuda_device).to(dt)
        nw = (1 + 0.1 * torch.randn(H, device=cuda_device)).to(dt)
        r0 = resid.float().clone()
        x_next = torch.empty((B, H), dtype=dt, device=cuda_device)
        ops.mlp_dense(x, layer.wg, layer.wu, wd, layer.threshold, resid=resid, x_next=x_next,
                      norm_weight=nw, eps=1e-5)
        assert O.rel_l2(to_np(resid), to_np(r0 + plain.float())) <= 5e-3
        rr = resid.float()
        y = (rr * torch.rsqrt(rr.pow(2).mean(-1, keepdim=True) + 1e-5)).to(dt)
        assert O.rel_l2(to_np(x_next), to_np(nw.float() * y.float())) <= 5e-3
    # the sparse path on the same workspace afterwards: the dense path left it clean
    sparse = ops.mlp(x[:4].contiguous(), layer.wg, layer.wu, layer.wdt, layer.threshold)
    assert O.rel_l2(to_np(sparse), to_np(plain[:4].reshape(4, 1, H))) <= 2e-2


def test_unsupported_shapes_are_refused(cuda_device):
    from cats_b200 import _lib, ops

    assert not ops.dense_supported(4, 1000, 2752, torch.float16)      # H not a multiple of 128
    assert not ops.dense_supported(4, 1024, 2700, torch.float16)      # I not a multiple of 64
    assert not ops.dense_supported(4, 1024, 2752, torch.float32)
    x = torch.zeros((4, 1024), device=cuda_device)
    w = torch.zeros((2752, 1024), device=cuda_device)
    wd = torch.zeros((1024, 2752), device=cuda_device)
    with pytest.raises(RuntimeError, match="unsupported mode"):
        ops.mlp_dense(x, w, w, wd, 0.1)


@pytest.mark.parametrize("B,dt", [(8, torch.float16), (3, torch.bfloat16)])
def test_stack_on_the_dense_path_matches_the_oracle_chain(B, dt, cuda_device):
    from cats_b200 import synth
    from cats_b200.stack import CatsMLPStack

    H, I, L = 4096, 14336, 2
    layers = synth.make_stack(L, H, I, dt, cuda_device, 23, 0.5)
    stack = CatsMLPStack(layers, batch=B)              # the switch picks the dense path here
    assert stack.dense
    bf16 = lambda a: torch.from_numpy(np.asarray(a, np.float32)).to(torch.bfloat16).float().numpy()
    rnd = np.float16 if dt == torch.float16 else bf16
    for seed in (1, 2):                                  # graph replay with a new input
        x0 = synth.make_x(B, H, dt, cuda_device, seed).reshape(B, H)
        stack.set_input(x0)
        stack.run_device()
        torch.cuda.synchronize()
        assert stack.ws.counters()[1] == 0
        xe, re_, _ = O.mlp_stack(to_np(x0), [(to_np(l.wg), to_np(l.wu), to_np(l.wdt).T) for l in layers],
                                 [l.threshold for l in layers], round_to=rnd)
        tol = 2e-2 if dt == torch.float16 else 5e-2
        assert O.rel_l2(to_np(stack.resid), re_) <= tol
        assert O.rel_l2(to_np(stack.x), xe) <= tol




@pytest.mark.gpu
def test_the_switch_follows_batch_and_density():
    from cats_b200 import ops

    assert not ops.use_dense(1)
    assert ops.use_dense(2) and ops.use_dense(4) and ops.use_dense(16)       # 50 %: union >= 0.75
    assert not ops.use_dense(2, sparsity=0.7) and ops.use_dense(4, sparsity=0.7)
    assert not ops.use_dense(4, sparsity=0.9) and ops.use_dense(8, sparsity=0.9)
    assert not ops.use_dense(4, union_density=0.4) and ops.use_dense(3, union_density=0.9)
