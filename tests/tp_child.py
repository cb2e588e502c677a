"""torchrun child of tests/test_tp_gpu.py: a real IPC group running both compositions, several
steps back to back without host synchronisation in between (the parity buffers' job)."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from pipelink_b200 import tp  # noqa: E402


def _rel(ref, got):
    return float((got.double() - ref.double()).norm() / ref.double().norm())


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    m, n, k = 2048, 1024, 1024
    ms, nl, kl = m // world, n // world, k // world
    group = tp.IpcTpGroup(m, n, k, rank, world, dev)
    me = group.rank
    steps = 4
    gen = torch.Generator(device=dev).manual_seed(7)       # same stream of operands on every rank
    cases = []
    for _ in range(steps):
        a = torch.randn(m, k, generator=gen, device=dev).to(torch.bfloat16)
        b = (torch.randn(n, k, generator=gen, device=dev) * 0.1).to(torch.bfloat16)
        cases.append((a, b))
    # all-gather -> GEMM: the next shard is written while peers may still read the previous parity
    outs = []
    for a, b in cases:
        me.shard_view().copy_(a[rank * ms:(rank + 1) * ms])
        outs.append(me.ag(b[rank * nl:(rank + 1) * nl].contiguous()).clone())
    me.status.check("ag")
    for (a, b), o in zip(cases, outs):
        ref = a.float() @ b[rank * nl:(rank + 1) * nl].float().T
        assert _rel(ref, o) < 3e-3, "ag"
    dist.barrier()
    outs = []
    for a, b in cases:
        outs.append(me.rs(a[:, rank * kl:(rank + 1) * kl].contiguous(), b[:, rank * kl:(rank + 1) * kl].contiguous()).clone())
    me.status.check("rs")
    for (a, b), o in zip(cases, outs):
        ref = (a.float() @ b.float().T)[rank * ms:(rank + 1) * ms]
        assert torch.isfinite(o.float()).all() and _rel(ref, o) < 1e-2, "rs"
    dist.barrier()
    torch.cuda.synchronize()
    group.close()
    if rank == 0:
        print("TP CHILD OK")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
