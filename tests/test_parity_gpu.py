"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the reference's golden
vectors.  Bars: mask bit-exact except for gate values within 1e-3 (relative) of the threshold;
output relative L2 <= 1e-5 (fp32) / 1e-2 (fp16, bf16) against the fp32 oracle."""
import numpy as np
import pytest
import torch

from conftest import MLP_GOLDEN, load_golden
from oracle import cats_oracle as O

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}
OUT_TOL = {torch.float32: 1e-5, torch.float16: 1e-2, torch.bfloat16: 1e-2}


def to_np(t):
    return t.detach().float().cpu().numpy()


def run_and_check(x, wg, wu, wdt, thr, what="mlp"):
    """x (B,1,H); wg, wu, wdt (I,H) device tensors in the storage dtype.  Runs stage 1 with dense
    outputs and the whole MLP, checks both against the oracle evaluated on the same (rounded)
    values, and returns (out, n_flips)."""
    from cats_b200 import ops

    dt = x.dtype
    B, H = ops.batch_of(x)
    I = wg.shape[0]
    gate_dense = torch.empty((B, I), dtype=dt, device=x.device)
    flag = torch.zeros((B, I), dtype=torch.bool, device=x.device)
    ws = ops.gate(x, wg, thr, gate_dense=gate_dense, flag_dense=flag)
    n_active, status = ws.counters()
    out = ops.mlp(x, wg, wu, wdt, thr)
    assert out.shape == x.shape and out.dtype == dt
    torch.cuda.synchronize()

    xn, wgn, wun, wdn = to_np(x).reshape(B, H), to_np(wg), to_np(wu), to_np(wdt).T
    ref64 = O.dense_masked_mlp(xn, wgn, wun, wdn, thr, dtype=np.float64)
    kmask = flag.cpu().numpy()
    flips, outside = O.mask_band_check(ref64["post_act"], kmask, thr)
    assert outside == 0, f"{what}: {outside} mask differences outside the 1e-3 band"
    assert status == 0
    assert n_active == int(O.union_mask(kmask).sum())
    # gate values of every neuron, rounded to the storage dtype
    gd = to_np(gate_dense)
    assert O.rel_l2(gd, ref64["post_act"]) <= (1e-6 if dt == torch.float32 else 5e-3)
    ref32 = O.dense_masked_mlp(xn, wgn, wun, wdn, thr, dtype=np.float32,
                               mask=kmask if flips else None)
    err = O.rel_l2(to_np(out).reshape(B, H), ref32["out"])
    assert err <= OUT_TOL[dt], f"{what}: rel L2 {err:.3e} > {OUT_TOL[dt]:.0e}"
    return out, flips


def synth_case(H, I, B, dt, sparsity, seed, device):
    from cats_b200 import synth

    layer = synth.make_layer(H, I, dt, device, seed, sparsity=sparsity,
                             std=0.02 if H >= 1024 else 1.3 / np.sqrt(H))
    x = synth.make_x(B, H, dt, device, seed + 77)
    return x, layer


@pytest.mark.parametrize("name", [n for n in MLP_GOLDEN if "prefill" not in n])
def test_golden_vectors_of_the_reference(name, cuda_device):
    g = load_golden(name)
    dt = DT[str(g["dtype"])]
    dev = cuda_device
    x = torch.from_numpy(g["x"]).to(dev, dt)
    wg = torch.from_numpy(g["wg"]).to(dev, dt)
    wu = torch.from_numpy(g["wu"]).to(dev, dt)
    wdt = torch.from_numpy(g["wd"]).to(dev, dt).t().contiguous()
    thr = float(g["threshold"])
    out, flips = run_and_check(x, wg, wu, wdt, thr, name)
    if dt == torch.float32 and flips == 0:
        # the reference's own output for these inputs
        assert O.rel_l2(to_np(out), g["y"]) <= 1e-5
    elif flips == 0:
        assert O.rel_l2(to_np(out), g["y"]) <= 3e-2  # reference rounds every intermediate


@pytest.mark.parametrize("H,I", [(64, 32), (264, 100), (64, 1000), (1024, 2752), (4096, 11008),
                                 (4096, 14336), (8192, 28672)])
@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
def test_shapes_at_half_sparsity(H, I, dt, cuda_device):
    if H % 8 and dt != torch.float32:
        pytest.skip("rows must be whole 16-byte vectors")
    x, layer = synth_case(H, I, 1, dt, 0.5, 3, cuda_device)
    run_and_check(x, layer.wg, layer.wu, layer.wdt, layer.threshold, f"{H}x{I}")


@pytest.mark.parametrize("sparsity", [0.0, 0.3, 0.5, 0.7, 0.9, 1.0])
@pytest.mark.parametrize("dt", [torch.float32, torch.float16])
def test_sparsity_levels_including_empty_and_full(sparsity, dt, cuda_device):
    x, layer = synth_case(4096, 14336 if dt == torch.float16 else 11008, 1, dt, 0.5, 5, cuda_device)
    if sparsity == 0.0:
        thr = -1.0            # everything active (the reference sweeps thresholds from -1)
    elif sparsity == 1.0:
        thr = 1e9             # nothing active: the output must be exactly zero
    else:
        from cats_b200 import synth
        thr = synth.calibrate_threshold(layer.wg, sparsity, 99)
    out, _ = run_and_check(x, layer.wg, layer.wu, layer.wdt, thr, f"s={sparsity}")
    if sparsity == 1.0:
        assert float(out.abs().max()) == 0.0


@pytest.mark.parametrize("B", [1, 2, 3, 4, 5, 8, 13, 16])
@pytest.mark.parametrize("dt", [torch.float32, torch.float16, torch.bfloat16])
def test_batches_use_per_token_masks(B, dt, cuda_device):
    x, layer = synth_case(1024, 2752, B, dt, 0.7, 11 + B, cuda_device)
    run_and_check(x, layer.wg, layer.wu, layer.wdt, layer.threshold, f"B={B}")


def test_batch_at_model_shape(cuda_device):
    x, layer = synth_case(4096, 14336, 4, torch.float16, 0.5, 21, cuda_device)
    run_and_check(x, layer.wg, layer.wu, layer.wdt, layer.threshold, "mistral B=4")


def test_same_input_twice_gives_same_mask_and_list(cuda_device):
    from cats_b200 import ops

    x, layer = synth_case(4096, 14336, 1, torch.float16, 0.5, 31, cuda_device)
    I = layer.wg.shape[0]
    res = []
    for _ in range(2):
        flag = torch.zeros((1, I), dtype=torch.bool, device=cuda_device)
        ws = ops.gate(x, layer.wg, layer.threshold, flag_dense=flag)
        idx = torch.full((I,), -1, dtype=torch.int64, device=cuda_device)
        val = torch.zeros((I,), dtype=x.dtype, device=cuda_device)
        n = ops.export_list(ws, 1, x.dtype, idx, val)
        out = ops.mlp(x, layer.wg, layer.wu, layer.wdt, layer.threshold)
        res.append((flag.clone(), idx[:n].clone(), val[:n].clone(), out.clone()))
    assert torch.equal(res[0][0], res[1][0])
    assert torch.equal(res[0][1], res[1][1]) and torch.equal(res[0][2], res[1][2])
    # the list is ascending and equals the flagged positions
    assert torch.equal(res[0][1], torch.nonzero(res[0][0][0]).flatten())
    assert O.rel_l2(to_np(res[0][3]), to_np(res[1][3])) <= 1e-3


def test_stages_one_by_one_equal_the_fused_call(cuda_device):
    from cats_b200 import ops

    for dt in (torch.float32, torch.float16):
        x, layer = synth_case(1024, 2752, 2, dt, 0.5, 41, cuda_device)
        B, H, I = 2, 1024, 2752
        ws = ops.gate(x, layer.wg, layer.threshold)
        inter = torch.zeros((B, I), dtype=dt, device=cuda_device)
        ops.up(x, layer.wu, ws, inter_dense=inter)
        out3 = torch.empty((B, H), dtype=dt, device=cuda_device)
        ops.down(layer.wdt, ws, out3, B)
        fused = ops.mlp(x, layer.wg, layer.wu, layer.wdt, layer.threshold).reshape(B, H)
        assert O.rel_l2(to_np(out3), to_np(fused)) <= (1e-6 if dt == torch.float32 else 2e-3)
        ref = O.dense_masked_mlp(to_np(x).reshape(B, H), to_np(layer.wg), to_np(layer.wu),
                                 to_np(layer.wdt).T, layer.threshold)
        assert O.rel_l2(to_np(inter), ref["inter"]) <= (1e-5 if dt == torch.float32 else 5e-3)
        # dense (H, I) down projection fed with the scattered intermediate
        wd = layer.wdt.t().contiguous()
        dense = ops.down_dense(inter, wd)
        assert O.rel_l2(to_np(dense), ref["out"]) <= OUT_TOL[dt]
        # fp32 accumulate convention of the reference's atomic ops: out += result
        acc = torch.ones((B, H), dtype=torch.float32, device=cuda_device)
        ws = ops.gate(x, layer.wg, layer.threshold)
        ops.updown(x, layer.wu, layer.wdt, ws, out=acc, accumulate_f32=True)
        assert O.rel_l2(to_np(acc) - 1.0, ref["out"]) <= OUT_TOL[dt]


def test_lists_left_by_an_earlier_call_are_never_read(cuda_device):
    """The kernels keep their active lists in the workspace between stages.  A call must only read
    lists it wrote itself: overwrite them with garbage between calls (and change the batch size,
    which changes their layout) and the results must not move.  The accumulators and the header
    (which must stay clean between calls) are left alone."""
    from cats_b200 import ops

    dev, dt = cuda_device, torch.float16
    up = lambda v: (v + 255) // 256 * 256
    for H, I in [(64, 160), (64, 1000), (1024, 2752), (4096, 14336)]:
        ws = ops.get_workspace(dev, H, I)
        # workspace layout (cats_common.cuh, ws_layout): header, segment counts, accumulators,
        # then the list arrays; every array starts on a 256-byte boundary
        o_cnt = 256
        o_acc = o_cnt + 4 * 1024
        o_idx = up(o_acc + 4 * 2 * 16 * H)
        o_gate = up(o_idx + 4 * I)
        o_flat = up(o_gate + 4 * I * 16)
        o_h = up(o_flat + 4 * I)
        o_end = up(o_h + 4 * I * 16)
        assert o_end + 48 * 1024 == ws.nbytes          # + the dense stack kernel's table
        for B in (1, 2, 1, 4):
            x, layer = synth_case(H, I, B, dt, 0.5, 11 + B, dev)
            ref = O.dense_masked_mlp(to_np(x).reshape(B, H), to_np(layer.wg), to_np(layer.wu),
                                     to_np(layer.wdt).T, layer.threshold)
            for rep in range(3):
                ws.buf[o_cnt:o_acc].view(torch.int32).fill_(1 + rep)
                for lo, hi in ((o_idx, o_gate), (o_flat, o_h)):      # indices: a valid row
                    ws.buf[lo:hi].view(torch.int32).fill_(rep)
                for lo, hi in ((o_gate, o_flat), (o_h, o_end)):      # values: large
                    ws.buf[lo:hi].view(torch.float32).fill_(1000.0 * rep)
                out = ops.mlp(x, layer.wg, layer.wu, layer.wdt, layer.threshold, ws=ws)
                torch.cuda.synchronize()
                err = O.rel_l2(to_np(out).reshape(B, H), ref["out"])
                assert err <= 1e-2, (H, I, B, rep, err)
                n_active, status = ws.counters()
                assert status == 0
                assert abs(n_active - int(O.union_mask(ref["mask"]).sum())) <= 2, (H, I, B, rep)


def test_fused_residual_and_rmsnorm_tail(cuda_device):
    from cats_b200 import ops

    for dt in (torch.float32, torch.float16, torch.bfloat16):
        x, layer = synth_case(1024, 2752, 2, dt, 0.5, 51, cuda_device)
        B, H = 2, 1024
        resid = torch.randn((B, H), device=cuda_device).to(dt)
        nw = (1 + 0.1 * torch.randn(H, device=cuda_device)).to(dt)
        r0 = to_np(resid)
        x_next = torch.empty((B, H), dtype=dt, device=cuda_device)
        plain = ops.mlp(x, layer.wg, layer.wu, layer.wdt, layer.threshold).reshape(B, H)
        ops.mlp(x, layer.wg, layer.wu, layer.wdt, layer.threshold, resid=resid, x_next=x_next,
                norm_weight=nw, eps=1e-5)
        r_exp = torch.from_numpy(r0).to(cuda_device) + plain.float()
        assert O.rel_l2(to_np(resid), to_np(r_exp)) <= (1e-6 if dt == torch.float32 else 5e-3)
        rr = resid.float()
        y = (rr * torch.rsqrt(rr.pow(2).mean(-1, keepdim=True) + 1e-5)).to(dt)
        x_exp = (nw.float() * y.float())
        assert O.rel_l2(to_np(x_next), to_np(x_exp)) <= (1e-6 if dt == torch.float32 else 5e-3)


def test_mlp_stack_matches_oracle_chain(cuda_device):
    import ctypes
    from cats_b200 import _lib, ops, synth

    dt, H, I, L, B = torch.float16, 1024, 2752, 5, 1
    layers = synth.make_stack(L, H, I, dt, cuda_device, 7, 0.5)
    x0 = synth.make_x(B, H, dt, cuda_device, 123).reshape(B, H)
    x_io, x_tmp, resid = x0.clone(), torch.empty_like(x0), x0.clone()
    ws = ops.get_workspace(cuda_device, H, I)
    arr = lambda ts: (ctypes.c_void_p * L)(*[t.data_ptr() for t in ts])
    thr = (ctypes.c_float * L)(*[l.threshold for l in layers])
    st = _lib.lib().cats_mlp_stack(L, arr([l.wg for l in layers]), arr([l.wu for l in layers]),
                                   arr([l.wdt for l in layers]), thr, x_io.data_ptr(),
                                   x_tmp.data_ptr(), resid.data_ptr(), ws.ptr, ws.nbytes, B, H, I,
                                   _lib.F16, 1e-6, torch.cuda.current_stream().cuda_stream)
    _lib.check(st)
    torch.cuda.synchronize()
    xe, re_, counts = O.mlp_stack(to_np(x0), [(to_np(l.wg), to_np(l.wu), to_np(l.wdt).T)
                                              for l in layers], [l.threshold for l in layers],
                                  round_to=np.float16)
    assert O.rel_l2(to_np(resid), re_) <= 1e-2
    assert O.rel_l2(to_np(x_io), xe) <= 1e-2


def test_flash_gemv_operator_api(cuda_device):
    """Every reference operator name, with the reference's layouts (flash_gemv/test/
    test_fuse_gemv_cmp.py builds its inputs the same way)."""
    import flash_gemv as fg

    dev, dt = cuda_device, torch.float16
    x, layer = synth_case(1024, 2752, 1, dt, 0.5, 61, dev)
    B, H, I = 1, 1024, 2752
    thr = layer.threshold
    wg, wu, wdt = layer.wg, layer.wu, layer.wdt
    wd = wdt.t().contiguous()                      # (H, I) nn.Linear layout
    ref = O.dense_masked_mlp(to_np(x).reshape(B, H), to_np(wg), to_np(wu), to_np(wd), thr)
    ok = lambda t, tol=1e-2: O.rel_l2(to_np(t).reshape(B, -1), ref["out"]) <= tol

    for fn in (fg.flag_gemv_gemv_inner, torch.ops.flash_gemv.flag_gemv_gemv_inner):
        y = fn(x, wg, wu, wd, thr)
        assert y.shape == x.shape and ok(y)
    with pytest.raises(RuntimeError):
        fg.flag_gemv_gemv_inner_bf16(x, wg, wu, wd, thr)     # dtype mismatch is an error
    assert ok(fg.flag_gemv_gemv_inner_bf16(x.bfloat16(), wg.bfloat16(), wu.bfloat16(),
                                           wd.bfloat16(), thr), 3e-2)
    assert ok(fg.flag_gemv_gemv_inner_fp32(x.float(), wg.float(), wu.float(), wd.float(), thr),
              1e-5)
    out = torch.empty((1, B, H), dtype=dt, device=dev)
    fg.flag_gemv_gemv(x, wg, wu, wd, out, thr)
    assert ok(out)
    for fn in (fg.flag_gemv_gemv_atomic, fg.fuse_gemv_gemv_gemv):
        acc = torch.zeros((1, B, H), dtype=torch.float32, device=dev)
        fn(x, wg, wu, wdt, acc, thr)
        assert ok(acc)
    acc = torch.zeros((1, B, H), dtype=torch.float32, device=dev)
    flag = torch.zeros((1, B, I), dtype=torch.bool, device=dev)
    fg.fuse_gemv_flag_gemv_gemv(x, wg, wu, wdt, acc, flag, thr)
    assert ok(acc) and np.array_equal(flag.cpu().numpy().reshape(B, I), ref["mask"])

    # stage ops
    val = torch.empty((1, B, I), dtype=dt, device=dev)
    for fn in (fg.fuse_gemv_flag_local, fg.fuse_gemv_flag, fg.fuse_gemv_flag_batch):
        flag.zero_()
        fn(x, wg, val, flag, thr)
        assert np.array_equal(flag.cpu().numpy().reshape(B, I), ref["mask"])
        assert O.rel_l2(to_np(val).reshape(B, I), ref["post_act"]) <= 5e-3
    fg.fuse_flag_gemv_local(x, wu, val, flag)          # in place: gate -> gate * up
    assert O.rel_l2(to_np(val).reshape(B, I), ref["inter"]) <= 5e-3
    acc = torch.zeros((1, B, H), dtype=torch.float32, device=dev)
    fg.atomic_gemv(val, wdt, acc, flag)
    assert ok(acc)
    inter = torch.zeros((1, B, I), dtype=dt, device=dev)
    flag.zero_()
    fg.fuse_gemv_flag_gemv(x, wg, wu, inter, flag, thr)
    assert O.rel_l2(to_np(inter).reshape(B, I), ref["inter"]) <= 5e-3
    idx = torch.zeros(I, dtype=torch.int64, device=dev)
    vals = torch.zeros((1, 1, I), dtype=dt, device=dev)
    n = fg.fuse_gemv_cmp(x, wg, vals, idx, thr)
    assert n == int(ref["mask"].sum())
    assert np.array_equal(idx[:n].cpu().numpy(), np.nonzero(ref["mask"][0])[0])

    # the names the reference backs with Triton: Wgate is (H, I), x_1 is the precomputed gate
    wgate_hi = wg.t().contiguous()
    x_1 = torch.nn.functional.silu(torch.nn.functional.linear(x, wg))
    assert ok(fg.gemv_gemv_triton(x, x_1, wu, wdt, thr), 2e-2)
    assert ok(fg.flag_gemv_gemv_triton(x, wgate_hi, wu, wdt, thr))
    x2 = x.reshape(1, H)
    for fn in (fg.flag_gemv_gemv_dejavu, fg.flag_gemv_gemv_fuse_dejavu):
        y = fn(x2, wgate_hi, wu, wdt, thr)
        assert y.shape == (1, H) and ok(y)


def test_module_decode_runs_cuda_path_and_matches_dense_branch(cuda_device):
    from cats_b200 import sparse_silu as S

    for cls, dt in ((S.LlamaSparseSiluMLP, torch.float16), (S.MistralSparseSiluMLP, torch.bfloat16),
                    (S.LlamaSparseSiluMLP, torch.float32)):
        torch.manual_seed(0)
        m = cls({"hidden_size": 1024, "intermediate_size": 2752}).to(cuda_device, dt)
        with torch.no_grad():
            for lin in (m.gate_proj, m.up_proj, m.down_proj):
                lin.weight.normal_(0, 0.04)
        x = torch.randn(2, 1, 1024, device=cuda_device).to(dt)
        m.is_profile = True
        m.dead_threshold = torch.tensor(0.25)
        with torch.no_grad():
            m.sp_method = 0
            dense = m(x)
            m.sp_method = 1
            y1 = m(x)
            m.sp_method = 2
            m.wdown_t = m.down_proj.weight.t().contiguous()
            y2 = m(x)
            assert y1.shape == x.shape and y1.dtype == dt
            tol = 1e-4 if dt == torch.float32 else 3e-2
            assert O.rel_l2(to_np(y1), to_np(dense)) <= tol
            assert O.rel_l2(to_np(y2), to_np(dense)) <= tol
            xp = torch.randn(2, 7, 1024, device=cuda_device).to(dt)
            assert m(xp).shape == xp.shape       # prefill: dense branch


def test_bad_arguments_raise(cuda_device):
    from cats_b200 import ops

    x, layer = synth_case(64, 32, 1, torch.float16, 0.5, 71, cuda_device)
    with pytest.raises(RuntimeError, match="dtype"):
        ops.mlp(x, layer.wg.float(), layer.wu, layer.wdt, 0.1)
    with pytest.raises(RuntimeError, match="contiguous"):
        ops.mlp(x, layer.wg.t().contiguous().t(), layer.wu, layer.wdt, 0.1)
    with pytest.raises(RuntimeError, match="batch"):
        ops.mlp(x.expand(17, 1, 64).contiguous(), layer.wg, layer.wu, layer.wdt, 0.1)
    with pytest.raises(RuntimeError):
        ops.mlp(x, layer.wg, layer.wu[:16].contiguous(), layer.wdt, 0.1)
