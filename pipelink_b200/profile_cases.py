"""Small, self-terminating cases of each hot kernel, sized for a profiler capture.

``python -m pipelink_b200.profile_cases decode``     16 layers, vocab 128256, 4 tokens at position 4096
``python -m pipelink_b200.profile_cases attention``  causal prefill, S=8192, 32 query / 8 KV heads, d=128
``python -m pipelink_b200.profile_cases moe``        MoE forward, 4096 tokens of the headline shape

``torchrun --nproc-per-node N -m pipelink_b200.profile_cases ep-phases``
                                                     device time of every phase of the expert-parallel forward
                                                     (CUDA events; a timing tool, not a profiler case)

Each case holds a few GB on the device at most, touches more than the L2 holds, and launches the
kernel of interest a handful of times.
"""
from __future__ import annotations

import sys

import torch


def decode_case(dev):
    from . import decode as hd
    torch.manual_seed(0)
    L, V = 16, 128256
    mk = lambda *s: (torch.randn(*s, device=dev) * 0.02).to(torch.bfloat16)
    ones = lambda *s: torch.ones(*s, device=dev)
    w = dict(qkv_w=mk(L, hd.QKV_ROWS, hd.HIDDEN), o_w=mk(L, hd.HIDDEN, hd.HIDDEN), up_w=mk(L, hd.FFN, hd.HIDDEN),
             gate_w=mk(L, hd.FFN, hd.HIDDEN), down_w=mk(L, hd.HIDDEN, hd.FFN), attn_norm=ones(L, hd.HIDDEN),
             mlp_norm=ones(L, hd.HIDDEN), lm_norm=ones(hd.HIDDEN), lm_head=mk(V, hd.HIDDEN))
    s = hd.DecodeSession(w, max_seq_len=4096 + 16, device=dev)
    s.k_cache[:, :4096].normal_()
    s.v_cache[:, :4096].normal_()
    s.start(1, 4096)
    s.decode(4)
    print("tokens", s.token_out[4097:4101].tolist())


def attention_case(dev, seq=8192):
    from . import attention as att
    torch.manual_seed(0)
    q = torch.randn(1, seq, 32, 128, device=dev).to(torch.bfloat16)
    k = torch.randn(1, seq, 8, 128, device=dev).to(torch.bfloat16)
    v = torch.randn(1, seq, 8, 128, device=dev).to(torch.bfloat16)
    for _ in range(3):
        out, _ = att.attention_fwd(q, k, v)
    torch.cuda.synchronize()
    print("attention ok", float(out.float().abs().mean()))


def moe_case(dev, tokens=4096):
    from . import mok
    shape = mok.Shape("profile", 64, 4096, 2048, 8, tokens)
    torch.manual_seed(0)
    E, H, I = shape.experts, shape.hidden, shape.intermediate
    mk = lambda *s: (torch.randn(*s, device=dev) * 0.02).to(torch.bfloat16)
    host = mok.MoKHost(shape)
    host.load_weights(mk(E, I, H), mk(E, I, H), mk(E, H, I))
    inputs = mok.MoKHost.new_inputs(shape, 1, dev)
    for _ in range(3):
        out = host.forward(inputs)["output"]
    torch.cuda.synchronize()
    print("moe ok", float(out.float().abs().mean()))


def ep_phases_case(tokens=8192, steps=10):
    """One rank per GPU under torchrun. Prints, for each phase of the expert-parallel forward step at
    the headline expert shape, the mean / min / max over ranks of its device time."""
    import os

    import torch.distributed as dist

    from . import ep, mok
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    base = mok.CONFIG2
    shape = mok.Shape("ep-phases", base.experts, base.hidden, base.intermediate, base.topk, tokens)
    session = ep.BenchSession(shape, dev, rank, world)
    h = session.host
    phases = [("quantise", h.quantize_tokens), ("publish routes", h.publish_routes), ("barrier", h.barrier),
              ("schedule", h.build_schedule), ("pull", h.pull), ("gate/up GEMM", h.gemm_gate_up),
              ("down GEMM + push", h.gemm_down_push), ("barrier ", h.barrier), ("epilogue", h.fwd_epilogue)]
    for _ in range(5):
        session.step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    acc = [0.0] * len(phases)
    for _ in range(steps):
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(phases) + 1)]
        evs[0].record()
        for i, (_, fn) in enumerate(phases):
            fn()
            evs[i + 1].record()
        torch.cuda.synchronize()
        for i in range(len(phases)):
            acc[i] += evs[i].elapsed_time(evs[i + 1]) / steps
    mine = torch.tensor(acc, device=dev)
    every = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(every, mine)
    h.status.check("ep-phases")
    if rank == 0:
        m = torch.stack(every).cpu()
        print(f"world {world}, tokens per rank {tokens}, rows on rank 0: {int(h.schedule.num_tokens.item())}")
        for i, (name, _) in enumerate(phases):
            print(f"{name:18s} mean {m[:, i].mean():.3f}  min {m[:, i].min():.3f}  max {m[:, i].max():.3f} ms")
        print(f"{'sum of means':18s} {float(m.mean(0).sum()):.3f} ms")
    dist.barrier()
    session.group.close()
    dist.destroy_process_group()


def main(argv):
    if len(argv) >= 2 and argv[1] == "ep-phases":
        if not torch.cuda.is_available():
            raise SystemExit("profile_cases needs a CUDA device")
        return ep_phases_case()
    if len(argv) < 2 or argv[1] not in ("decode", "attention", "moe"):
        raise SystemExit(__doc__)
    if not torch.cuda.is_available():
        raise SystemExit("profile_cases needs a CUDA device")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    {"decode": decode_case, "attention": attention_case, "moe": moe_case}[argv[1]](dev)


if __name__ == "__main__":
    main(sys.argv)
