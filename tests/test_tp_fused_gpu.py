"""The tensor-parallel persistent kernel (cats_tp_mlp_stack): on one GPU with the exchange running
against the rank's own buffer, and on two GPUs (child processes, one per GPU) when the box has
them.  No test here makes a rank fail inside a kernel; a missing peer is only ever simulated on
the host side (bad arguments)."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import cats_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def to_np(t):
    return t.detach().float().cpu().numpy()


@pytest.mark.parametrize("H,I,L,B,dt", [(1024, 2752, 5, 1, torch.float16),
                                        (4096, 14336, 3, 2, torch.bfloat16),
                                        (2048, 4096, 4, 4, torch.float32),
                                        # a rank's slice of an 8-way split: 12 rows per CTA, one
                                        # part per layer, every CTA on its own rows' list
                                        (4096, 1792, 6, 1, torch.float16),
                                        (1024, 1792, 4, 2, torch.float32)])
def test_single_rank_exchange_matches_the_plain_stack_and_the_oracle(H, I, L, B, dt, cuda_device):
    from cats_b200 import synth, tp
    from cats_b200.stack import CatsMLPStack

    layers = synth.make_stack(L, H, I, dt, cuda_device, 7, 0.5)
    x0 = synth.make_x(B, H, dt, cuda_device, 123).reshape(B, H)
    fused = tp.FusedTPStack(layers, batch=B)          # world size 1: own exchange buffer only
    for _ in range(3):                                 # the slot sets alternate across launches
        fused.set_input(x0)
        fused.run_device()
    torch.cuda.synchronize()
    assert fused.device_status() == 0
    plain = CatsMLPStack(layers, batch=B)
    plain.set_input(x0)
    plain.run_device()
    torch.cuda.synchronize()
    # fp32 sums in a different order; 16-bit storage rounds them differently now and then and a
    # gate value next to the threshold may then flip in a later layer
    # (bf16 keeps 8 bits: over three layers a few flipped gates move the result by a few percent)
    tight = {torch.float32: 1e-5, torch.float16: 2e-2, torch.bfloat16: 5e-2}[dt]
    assert O.rel_l2(to_np(fused.resid), to_np(plain.resid)) <= tight
    assert O.rel_l2(to_np(fused.x), to_np(plain.x)) <= tight
    bf16 = lambda a: torch.from_numpy(np.asarray(a, np.float32)).to(torch.bfloat16).float().numpy()
    rnd = {torch.float16: np.float16, torch.float32: None, torch.bfloat16: bf16}[dt]
    xe, re_, _ = O.mlp_stack(to_np(x0), [(to_np(l.wg), to_np(l.wu), to_np(l.wdt).T) for l in layers],
                             [l.threshold for l in layers], round_to=rnd)
    tol = {torch.float32: 1e-3, torch.float16: 2e-2, torch.bfloat16: 5e-2}[dt]
    assert O.rel_l2(to_np(fused.resid), re_) <= tol
    assert O.rel_l2(to_np(fused.x), xe) <= tol
    fused.close()


def test_bad_rank_arguments_are_refused_on_the_host(cuda_device):
    from cats_b200 import _lib, ops, synth

    H, I, L, B, dt = 1024, 2752, 2, 1, torch.float16
    layers = synth.make_stack(L, H, I, dt, cuda_device, 3, 0.5)
    x = synth.make_x(B, H, dt, cuda_device, 1).reshape(B, H)
    resid = x.clone()
    ws = ops.get_workspace(cuda_device, H, I)
    lib = _lib.lib()
    xb = torch.zeros(lib.cats_tp_exchange_bytes(H), dtype=torch.uint8, device=cuda_device)
    arr = lambda ts: (ctypes.c_void_p * L)(*[t.data_ptr() for t in ts])
    thr = (ctypes.c_float * L)(*[l.threshold for l in layers])

    def call(nranks, rank, ptrs, batch=B):
        ex = (ctypes.c_void_p * max(1, len(ptrs)))(*ptrs)
        return lib.cats_tp_mlp_stack(L, arr([l.wg for l in layers]), arr([l.wu for l in layers]),
                                     arr([l.wdt for l in layers]), thr, x.data_ptr(),
                                     resid.data_ptr(), ws.ptr, ws.nbytes, batch, H, I, _lib.F16, 1e-6,
                                     nranks, rank, ex, torch.cuda.current_stream().cuda_stream)

    assert call(0, 0, [xb.data_ptr()]) == _lib.ERR_SHAPE
    assert call(9, 0, [xb.data_ptr()] * 9) == _lib.ERR_SHAPE
    assert call(2, 2, [xb.data_ptr()] * 2) == _lib.ERR_SHAPE
    assert call(2, 0, [xb.data_ptr(), None]) == _lib.ERR_NULL       # a peer that was never mapped
    assert call(1, 0, [xb.data_ptr() + 16]) == _lib.ERR_ALIGN
    assert call(1, 0, [xb.data_ptr()], batch=5) == _lib.ERR_SHAPE
    assert call(1, 0, [xb.data_ptr()]) == _lib.OK
    torch.cuda.synchronize()
    assert ws.counters()[1] == 0
    # the same workspace serves the other entry points afterwards (its barrier counters and
    # accumulators are left consistent whichever schedule the tensor-parallel launch took)
    from oracle import cats_oracle as O2
    out = ops.mlp(x.reshape(B, 1, H), layers[0].wg, layers[0].wu, layers[0].wdt, layers[0].threshold, ws=ws)
    ref = O2.dense_masked_mlp(to_np(x), to_np(layers[0].wg), to_np(layers[0].wu), to_np(layers[0].wdt).T,
                              layers[0].threshold)
    assert O2.rel_l2(to_np(out).reshape(B, H), ref["out"]) <= 1e-2
    assert ws.counters()[1] == 0


def test_a_wait_that_runs_out_ends_the_kernel_with_a_status_and_recovery_works(cuda_device):
    """Rank 0 of a pretended group of two, on one GPU: the second exchange buffer is a local
    buffer that nobody writes, so rank 0's wait for rank 1's partial sums can only run out.  With
    the limit set to 50 ms (waits for other ranks get four times that) the kernel must end by
    itself, leave a non-zero device status, and - after the documented recovery: new exchange
    buffers, cleared workspace - the next call must be correct.  Nothing faults and nothing
    spins for ever: this is the bounded-wait path doing its job."""
    from cats_b200 import _lib, ops, synth, tp
    from cats_b200.stack import CatsMLPStack

    H, I, L, B, dt = 1024, 2752, 3, 1, torch.float16
    layers = synth.make_stack(L, H, I, dt, cuda_device, 5, 0.5)
    x0 = synth.make_x(B, H, dt, cuda_device, 77).reshape(B, H)
    lib = _lib.lib()
    ws = ops.Workspace(cuda_device, H, I)
    own = torch.zeros(lib.cats_tp_exchange_bytes(H), dtype=torch.uint8, device=cuda_device)
    silent = torch.zeros_like(own)                       # "rank 1": never written by anyone
    arr = lambda ts: (ctypes.c_void_p * L)(*[t.data_ptr() for t in ts])
    thr = (ctypes.c_float * L)(*[l.threshold for l in layers])
    x, resid = x0.clone(), x0.clone()
    ex = (ctypes.c_void_p * 2)(own.data_ptr(), silent.data_ptr())
    assert lib.cats_set_option(b"wait_ms", 50) == 0
    try:
        import time
        t0 = time.time()
        st = lib.cats_tp_mlp_stack(L, arr([l.wg for l in layers]), arr([l.wu for l in layers]),
                                   arr([l.wdt for l in layers]), thr, x.data_ptr(), resid.data_ptr(),
                                   ws.ptr, ws.nbytes, B, H, I, _lib.F16, 1e-6, 2, 0, ex,
                                   torch.cuda.current_stream().cuda_stream)
        assert st == _lib.OK                              # asynchronous: the launch itself is fine
        n_active, status = ws.counters()                  # synchronises the stream
        elapsed = time.time() - t0
    finally:
        assert lib.cats_set_option(b"wait_ms", 1000) == 0
    assert status == 3, status                            # STATUS_WAIT_TIMEOUT_MEGA
    assert elapsed < 5.0, elapsed                         # ended by itself, well inside a few limits
    # recovery as documented in include/cats_b200.h: the workspace is cleared, new buffers
    _lib.check(lib.cats_workspace_init(ws.ptr, ws.nbytes, torch.cuda.current_stream().cuda_stream))
    fused = tp.FusedTPStack(layers, batch=B)              # fresh exchange buffer, world size 1
    fused.ws = ws
    fused.set_input(x0)
    fused.run_device()
    torch.cuda.synchronize()
    assert fused.device_status() == 0
    plain = CatsMLPStack(layers, batch=B)
    plain.set_input(x0)
    plain.run_device()
    torch.cuda.synchronize()
    assert O.rel_l2(to_np(fused.resid), to_np(plain.resid)) <= 2e-2
    fused.close()


def test_a_stack_that_saw_a_timeout_refuses_further_launches(cuda_device):
    from cats_b200 import synth, tp

    layers = synth.make_stack(2, 1024, 2752, torch.float16, cuda_device, 5, 0.5)
    fused = tp.FusedTPStack(layers, batch=1)
    fused.ws.buf[8:12].view(torch.int32).fill_(3)         # the status word, as a time-out leaves it
    with pytest.raises(RuntimeError, match="bounded wait"):
        fused.check()
    with pytest.raises(RuntimeError, match="invalid"):
        fused.run_device()
    fused.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_on_two_gpus_match_the_unsharded_oracle():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29541",
           os.path.join(ROOT, "tests", "tp_fused_worker.py")]
    res = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "TP_FUSED_OK" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]
