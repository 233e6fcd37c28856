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
