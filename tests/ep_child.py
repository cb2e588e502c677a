"""torchrun child of tests/test_ep_gpu.py: a real IPC group, checked against the CPU oracle."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from oracle import moe as omoe  # noqa: E402
from pipelink_b200 import ep, mok  # noqa: E402


def _f(t):
    return t.detach().float().cpu().numpy()


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    shape = mok.Shape("ep-child", 8 * world, 512, 256, 2, 256)
    torch.manual_seed(0)  # same weights on every rank; each keeps its slice
    E, H, I = shape.experts, shape.hidden, shape.intermediate
    wg = (torch.randn(E, I, H, device=dev) * 0.02).to(torch.bfloat16)
    wu = (torch.randn(E, I, H, device=dev) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device=dev) * 0.02).to(torch.bfloat16)
    group = ep.IpcGroup(shape, rank, world, dev)
    host = ep.EpMoKHost(shape, rank, group)
    El = E // world
    host.load_weights(wg[rank * El:(rank + 1) * El], wu[rank * El:(rank + 1) * El], wd[rank * El:(rank + 1) * El])
    for generation in (1, 2, 3):
        inputs = [mok.MoKHost.new_inputs(shape, generation, dev, rank=r, world=world) for r in range(world)]
        out = _f(host.forward(inputs[rank])["output"])
        weights = omoe.quantize_weights(_f(wg), _f(wu), _f(wd))
        ref = omoe.forward_multi_rank([_f(i.x) for i in inputs], [i.experts.cpu().numpy().astype(np.int32) for i in inputs],
                                      [i.router.cpu().numpy() for i in inputs], weights, world,
                                      padding=mok.expert_padding())
        s = omoe.error_stats(ref["outputs"][rank], out)
        assert np.isfinite(out).all() and s["relative"] <= 2e-2, (rank, generation, s)
    torch.cuda.synchronize()
    dist.barrier()
    group.close()
    dist.destroy_process_group()
    if rank == 0:
        print("EP CHILD OK")


if __name__ == "__main__":
    main()
