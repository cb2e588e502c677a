"""torchrun child: a real context-parallel group over CUDA IPC; every rank's O and LSE must equal
the rows it owns of a single-GPU run of the same kernel (bitwise)."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from oracle import attention as oa  # noqa: E402
from pipelink_b200 import attention as att, ep  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    S, Hq, Hkv = 2048 * world, 8, 2
    mk = lambda n, role: torch.from_numpy(oa.philox_bf16(n, 9, role)).to(torch.bfloat16).to(dev)
    q, k, v = mk(S * Hq * 128, 1).reshape(S, Hq, 128), mk(S * Hkv * 128, 2).reshape(S, Hkv, 128), mk(S * Hkv * 128, 3).reshape(S, Hkv, 128)
    full_o, full_lse = att.attention_fwd(q[None], k[None], v[None])
    layout = att.CpRank.slab_layout(S, Hkv)
    slab = ep.IpcSlab(layout["nbytes"], rank, world)
    pos = torch.from_numpy(oa.zigzag_rows(S, world, rank)).to(dev)
    # the K/V exchange as a launch in front of the attention kernel, then inside it (gather warps)
    for fused in (False, True):
        r = att.CpRank(S, Hq, Hkv, rank, world, slab.ptrs, layout, dev, fused_push=fused)
        for step in range(3):
            o, lse = r.step(att.shard_zigzag(q, world, rank), att.shard_zigzag(k, world, rank), att.shard_zigzag(v, world, rank))
            torch.cuda.synchronize()
            r.status.check(f"cp step {step} (fused push: {fused})")
            assert torch.equal(o.view(torch.int16), full_o[0][pos].view(torch.int16)), (rank, step, fused)
            assert torch.equal(lse, full_lse[:, pos]), (rank, step, fused)
        torch.cuda.synchronize()
        dist.barrier()
    slab.close()
    dist.destroy_process_group()
    if rank == 0:
        print("CP CHILD OK")


if __name__ == "__main__":
    main()
