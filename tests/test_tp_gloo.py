"""Tensor-parallel host logic under gloo (2 CPU ranks): sharding bounds, slice algebra and the
all-reduce + tail sequence of ``TPStack``.  The CUDA kernels are replaced by a CPU restatement
through the ``local_mlp`` / ``tail`` hooks, so this checks exactly the part that is new relative
to the single-GPU path: that per-slice thresholding + a sum over ranks equals the unsharded MLP."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cats_b200 import synth, tp
from oracle import cats_oracle as O


def test_shard_bounds_cover_all_rows_in_multiples_of_32():
    for I in (32, 100, 11008, 14336, 28672):
        for world in (1, 2, 4, 8):
            edges = [tp.shard_bounds(I, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == I
            for (lo, hi), (lo2, _) in zip(edges, edges[1:]):
                assert hi == lo2 and lo <= hi
            assert all(lo % 32 == 0 for lo, _ in edges)
    with pytest.raises(RuntimeError):
        tp.shard_bounds(64, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_mlp(x, layer, out, ws=None):
    y = O.torch_dense_masked_mlp(x.float(), layer.wg.float(), layer.wu.float(),
                                 layer.wdt.t().float(), layer.threshold)
    out.copy_(y.reshape(out.shape).to(out.dtype))
    return out


def _cpu_tail(y, resid, x_next, eps):
    resid.add_(y)
    r = resid.float()
    x_next.copy_((r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + eps)).to(x_next.dtype))


def _worker(rank, world, port, H, I, L, B, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dev = torch.device("cpu")
        full = [synth.make_layer(H, I, torch.float32, dev, 50 + l, 0.5, std=1.3 / np.sqrt(H))
                for l in range(L)]
        x0 = synth.make_x(B, H, torch.float32, dev, 9).reshape(B, H)
        stack = tp.TPStack([tp.shard_layer(l, rank, world) for l in full], batch=B,
                           local_mlp=_cpu_mlp, tail=_cpu_tail)
        stack.set_input(x0)
        stack.run_device()
        # unsharded chain on every rank
        xe, re_, _ = O.mlp_stack(x0.numpy(), [(l.wg.numpy(), l.wu.numpy(), l.wdt.t().numpy())
                                              for l in full], [l.threshold for l in full])
        err_x, err_r = O.rel_l2(stack.x.numpy(), xe), O.rel_l2(stack.resid.numpy(), re_)
        # every rank ends with the same replicated state
        gathered = [torch.empty_like(stack.x) for _ in range(world)]
        dist.all_gather(gathered, stack.x)
        same = all(torch.equal(g, gathered[0]) for g in gathered)
        q.put((rank, err_x, err_r, same))
    finally:
        dist.destroy_process_group()


def test_tp_stack_two_ranks_equals_unsharded():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 256, 704, 3, 2, q))
             for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err_x, err_r, same in results:
        assert err_x < 1e-5 and err_r < 1e-5 and same, (rank, err_x, err_r, same)


# ---- failures, made on the host (no GPU involved) ----------------------------------------------
def _fault_worker(rank, world, port, case, q):
    import datetime
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=8))
    dev = torch.device("cpu")
    H, I, L, B = 64, 128, 3, 1
    full = [synth.make_layer(H, I, torch.float32, dev, 60 + l, 0.5, std=1.3 / np.sqrt(H))
            for l in range(L)]
    x0 = synth.make_x(B, H, torch.float32, dev, 9).reshape(B, H)
    t0 = time.monotonic()
    try:
        if case == "mismatched":
            # rank 1 was built with one layer fewer: it would run one all-reduce fewer
            mine = full if rank == 0 else full[:-1]
            tp.TPStack([tp.shard_layer(l, rank, world) for l in mine], batch=B,
                       local_mlp=_cpu_mlp, tail=_cpu_tail)
            q.put((rank, "no error", time.monotonic() - t0))
        elif case == "exits_before_a_step":
            stack = tp.TPStack([tp.shard_layer(l, rank, world) for l in full], batch=B,
                               local_mlp=_cpu_mlp, tail=_cpu_tail)
            store = dist.distributed_c10d._get_default_store()
            hb = tp.PeerHeartbeat(store, rank, world, deadline_s=2.0)
            stack.set_input(x0)
            stack.run_device()                      # step 0: everyone is there
            hb.beat(0)
            hb.require(0)
            if rank == 1:
                q.put((rank, "left", time.monotonic() - t0))
                q.close()
                q.join_thread()
                os._exit(0)                         # leaves between steps, nothing in flight
            t0 = time.monotonic()
            hb.beat(1)
            hb.require(1)                           # must raise: rank 1 never reports step 1
            q.put((rank, "no error", time.monotonic() - t0))
        elif case == "joins_late":
            store = dist.distributed_c10d._get_default_store()
            hb = tp.PeerHeartbeat(store, rank, world, deadline_s=6.0)
            if rank == 1:
                time.sleep(1.0)                     # late, but inside the deadline
            hb.beat(0)
            hb.require(0)
            q.put((rank, "ok", time.monotonic() - t0))
    except tp.PeerLost as e:
        q.put((rank, "PeerLost: " + str(e), time.monotonic() - t0))
    except RuntimeError as e:
        q.put((rank, "RuntimeError: " + str(e), time.monotonic() - t0))
    q.close()
    q.join_thread()                                 # the report is out before the process goes
    os._exit(0)                                     # no collective teardown with a missing peer


def _run_fault_case(case):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_fault_worker, args=(r, 2, port, case, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = {}
    for _ in range(2):
        rank, what, dt = q.get(timeout=120)
        out[rank] = (what, dt)
    for p in procs:
        p.join(timeout=60)
    return out


def test_ranks_that_disagree_on_the_stack_get_an_error_at_construction():
    out = _run_fault_case("mismatched")
    for rank in (0, 1):
        what, dt = out[rank]
        assert what.startswith("RuntimeError") and "layers" in what, out
        assert dt < 30


def test_a_rank_that_leaves_between_steps_is_noticed_on_the_host_within_the_deadline():
    out = _run_fault_case("exits_before_a_step")
    assert out[1][0] == "left"
    what, dt = out[0]
    assert what.startswith("PeerLost") and "[1]" in what, out
    assert dt < 10, dt                              # 2 s deadline, not a collective time-out


def test_a_rank_that_joins_late_but_in_time_is_waited_for():
    out = _run_fault_case("joins_late")
    assert out[0][0] == "ok" and out[1][0] == "ok", out
    assert out[0][1] >= 0.5                         # rank 0 really waited for rank 1


def test_heartbeat_on_a_local_store():
    store = dist.HashStore()
    a = tp.PeerHeartbeat(store, 0, 2, deadline_s=0.2)
    b = tp.PeerHeartbeat(store, 1, 2, deadline_s=0.2)
    a.beat(0)
    with pytest.raises(tp.PeerLost):
        a.require(0)                                # rank 1 has not reported yet
    b.beat(0)
    a.require(0)
    b.require(0)
    b.beat(3)
    a.require(2)                                    # a later step counts as well
