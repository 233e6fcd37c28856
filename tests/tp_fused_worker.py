"""Worker of the multi-GPU test of the fused tensor-parallel stack: one process per GPU (started by
torch.distributed.run), every rank runs FusedTPStack on its row slice and rank 0 compares the
result with the CPU oracle of the unsharded stack.  Prints ``TP_FUSED_OK`` on success."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from cats_b200 import synth, tp  # noqa: E402
from oracle import cats_oracle as O  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    to_np = lambda t: t.detach().float().cpu().numpy()
    ok = True
    for (H, I, L, B, dt) in [(1024, 3584, 5, 1, torch.float16), (4096, 14336, 3, 2, torch.bfloat16),
                             (2048, 4096, 4, 4, torch.float32)]:
        full = synth.make_stack(L, H, I, dt, dev, 7, 0.5)
        x0 = synth.make_x(B, H, dt, dev, 123).reshape(B, H)
        stack = tp.FusedTPStack([tp.shard_layer(l, rank, world) for l in full], batch=B)
        for rep in range(3):        # repeated launches reuse the exchange buffers
            stack.set_input(x0)
            stack.run_device()
        torch.cuda.synchronize()
        status = stack.device_status()
        xs, rs = [torch.empty_like(stack.x) for _ in range(world)], None
        dist.all_gather(xs, stack.x)
        same = all(torch.equal(xs[0], t) for t in xs)      # bit-identical on every rank
        if rank == 0:
            bf16 = lambda a: torch.from_numpy(np.asarray(a, np.float32)).to(torch.bfloat16).float().numpy()
            rnd = {torch.float16: np.float16, torch.float32: None, torch.bfloat16: bf16}[dt]
            xe, re_, _ = O.mlp_stack(to_np(x0), [(to_np(l.wg), to_np(l.wu), to_np(l.wdt).T)
                                                 for l in full], [l.threshold for l in full],
                                     round_to=rnd)
            tol = {torch.float32: 1e-3, torch.float16: 2e-2, torch.bfloat16: 5e-2}[dt]
            e_r, e_x = O.rel_l2(to_np(stack.resid), re_), O.rel_l2(to_np(stack.x), xe)
            print(f"H {H} I {I} L {L} B {B} {dt}: resid {e_r:.2e} x {e_x:.2e} status {status} "
                  f"identical {same}", flush=True)
            ok = ok and e_r <= tol and e_x <= tol and status == 0 and same
        stack.close()
        del full, stack
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, 0)
    if rank == 0 and int(flag.item()) == 1:
        print("TP_FUSED_OK", flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    os._exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
