"""Weight packing: HF state_dict -> kernel layout, the on-disk format, per-rank loading."""
import numpy as np
import pytest
import torch

from oracle import cats_oracle as O


def make_state_dict(L, H, I, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for i in range(L):
        p = f"model.layers.{i}.mlp."
        sd[p + "gate_proj.weight"] = (torch.randn(I, H, generator=g) * 0.1).to(dtype)
        sd[p + "up_proj.weight"] = (torch.randn(I, H, generator=g) * 0.1).to(dtype)
        sd[p + "down_proj.weight"] = (torch.randn(H, I, generator=g) * 0.1).to(dtype)
        sd[f"model.layers.{i}.input_layernorm.weight"] = torch.ones(H, dtype=dtype)
    return sd


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_pack_save_load_round_trip_and_rank_slices(dtype, tmp_path):
    from cats_b200 import pack, tp

    L, H, I = 3, 32, 160
    sd = make_state_dict(L, H, I, dtype)
    thr = [0.1, 0.2, 0.3]
    layers = pack.pack_state_dict(sd, thresholds=thr)
    assert len(layers) == L
    for i, l in enumerate(layers):
        p = f"model.layers.{i}.mlp."
        assert torch.equal(l.wg, sd[p + "gate_proj.weight"]) and torch.equal(l.wu, sd[p + "up_proj.weight"])
        assert torch.equal(l.wdt, sd[p + "down_proj.weight"].t()) and l.wdt.is_contiguous()
        assert l.threshold == pytest.approx(thr[i])
    path = str(tmp_path / "w.catspk")
    pack.save_packed(path, layers, meta={"model": "toy"})
    h = pack.read_header(path)
    assert (h["hidden"], h["intermediate"], h["layers"], h["meta"]) == (H, I, L, {"model": "toy"})
    assert all(off % 256 == 0 for trio in h["offsets"] for off in trio)
    back = pack.load_packed(path)
    for a, b in zip(layers, back):
        assert torch.equal(a.wg, b.wg) and torch.equal(a.wu, b.wu) and torch.equal(a.wdt, b.wdt)
        assert b.wg.dtype == dtype and a.threshold == pytest.approx(b.threshold)
    for world in (2, 3):
        for rank in range(world):
            part = pack.load_packed(path, rank=rank, world=world)
            direct = pack.pack_state_dict(sd, thresholds=thr, rank=rank, world=world)
            for a, b, c in zip(layers, part, direct):
                want = tp.shard_layer(a, rank, world)
                for x, y, z in ((want.wg, b.wg, c.wg), (want.wu, b.wu, c.wu), (want.wdt, b.wdt, c.wdt)):
                    assert torch.equal(x, y) and torch.equal(x, z)
    only = pack.load_packed(path, layers=[2])
    assert len(only) == 1 and torch.equal(only[0].wg, layers[2].wg)


def test_bad_files_and_shapes_are_refused(tmp_path):
    from cats_b200 import pack

    bad = tmp_path / "x.bin"
    bad.write_bytes(b"not a packed file at all")
    with pytest.raises(RuntimeError):
        pack.read_header(str(bad))
    with pytest.raises(RuntimeError):
        pack.pack_layer(torch.zeros(8, 4), torch.zeros(8, 4), torch.zeros(8, 4))
    with pytest.raises(RuntimeError):
        pack.pack_state_dict({"something.else": torch.zeros(1)})


@pytest.mark.gpu
def test_packed_state_dict_runs_the_cuda_path(cuda_device, tmp_path):
    from cats_b200 import ops, pack

    L, H, I, dt = 2, 1024, 2752, torch.float16
    sd = make_state_dict(L, H, I, dt, seed=5)
    layers = pack.pack_state_dict(sd, device=cuda_device, thresholds=[0.05] * L)     # GPU transpose
    path = str(tmp_path / "w.catspk")
    pack.save_packed(path, layers)
    loaded = pack.load_packed(path, device=cuda_device)
    x = torch.randn(1, 1, H, generator=torch.Generator().manual_seed(1)).to(cuda_device, dt)
    for i, (a, b) in enumerate(zip(layers, loaded)):
        assert torch.equal(a.wdt, b.wdt)
        out = ops.mlp(x, b.wg, b.wu, b.wdt, b.threshold)
        p = f"model.layers.{i}.mlp."
        f = lambda t: t.float().cpu().numpy()
        ref = O.dense_masked_mlp(f(x).reshape(1, H), f(sd[p + "gate_proj.weight"]), f(sd[p + "up_proj.weight"]),
                                 f(sd[p + "down_proj.weight"]), 0.05)
        assert O.rel_l2(f(out).reshape(1, H), ref["out"]) <= 1e-2
