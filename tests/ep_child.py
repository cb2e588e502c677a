"""torchrun child of tests/test_ep_gpu.py: a real IPC group. The forward is checked against the
CPU oracle; forward + backward against one rank holding every token and every expert (bitwise)."""
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
    shape = mok.Shape("ep-child", 8 * world, 512, 256, 2, 512)   # tokens * topk = 1024: the schedule writes stream positions
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
    # ---- host pipeline: three batches in flight give what one forward per batch gives
    batches = [mok.MoKHost.new_inputs(shape, g, dev, rank=rank, world=world) for g in (1, 2, 3)]
    want = [host.forward(b)["output"].clone().cpu() for b in batches]
    # ---- dispatch inside the gate/up GEMM (rows fetched from the peers under the mainloop): same bits
    host.fused_dispatch = True
    for b, w in zip(batches, want):
        got = host.forward(b)["output"].cpu()
        assert torch.equal(got.view(torch.int16), w.view(torch.int16)), (rank, "in-kernel dispatch")
    # ---- the FFN as ONE launch of the linked forward image (dispatch warps, both projections, combine push)
    from pipelink_b200 import moe_linked
    linked = moe_linked.LinkedMoE(host)
    for full in (False, True):      # full: the group barrier and the weighted epilogue inside the launch too
        host.attach_linked(linked, full=full)
        for fused in (True, False):
            host.fused_dispatch = fused
            for b, w in zip(batches, want):
                got = host.forward(b)["output"].cpu()
                assert torch.equal(got.view(torch.int16), w.view(torch.int16)), (rank, "one-launch forward", fused, full)
    host.attach_linked(None)
    host.fused_dispatch = False
    torch.cuda.synchronize()
    dist.barrier()
    linked.close()
    pin = lambda t: t.cpu().pin_memory()
    h_out = [torch.full((shape.tokens, H), float("nan"), dtype=torch.bfloat16).pin_memory() for _ in batches]
    pipe = ep.EpHostPipeline(host)
    for b, o in zip(batches, h_out):
        pipe.submit(pin(b.x), pin(b.experts.to(torch.int32)), pin(b.router), o)
    pipe.drain()
    host.status.check("EP host pipeline")
    for i, (o, w) in enumerate(zip(h_out, want)):
        assert torch.equal(o.view(torch.int16), w.view(torch.int16)), (rank, "pipeline", i)
    torch.cuda.synchronize()
    dist.barrier()
    group.close()

    # ---- receive streams: the same forward with the combine push written in arrival order
    group = ep.IpcGroup(shape, rank, world, dev, stream=True)
    host = ep.EpMoKHost(shape, rank, group)
    host.load_weights(wg[rank * El:(rank + 1) * El], wu[rank * El:(rank + 1) * El], wd[rank * El:(rank + 1) * El])
    assert host.stream_push and host.schedule_writes_streams
    for b, w in zip(batches, want):
        got = host.forward(b)["output"].cpu()
        assert torch.equal(got.view(torch.int16), w.view(torch.int16)), (rank, "receive streams")
    linked = moe_linked.LinkedMoE(host)
    host.fused_dispatch = True
    for full in (False, True):
        host.attach_linked(linked, full=full)
        for b, w in zip(batches, want):
            got = host.forward(b)["output"].cpu()
            assert torch.equal(got.view(torch.int16), w.view(torch.int16)), (rank, "one-launch forward, receive streams", full)
    host.attach_linked(None)
    host.fused_dispatch = False
    torch.cuda.synchronize()
    dist.barrier()
    linked.close()
    h_out = [torch.full((shape.tokens, H), float("nan"), dtype=torch.bfloat16).pin_memory() for _ in batches]
    pipe = ep.EpHostPipeline(host)
    for b, o in zip(batches, h_out):
        pipe.submit(pin(b.x), pin(b.experts.to(torch.int32)), pin(b.router), o)
    pipe.drain()
    host.status.check("EP host pipeline, receive streams")
    for i, (o, w) in enumerate(zip(h_out, want)):
        assert torch.equal(o.view(torch.int16), w.view(torch.int16)), (rank, "pipeline, receive streams", i)
    torch.cuda.synchronize()
    dist.barrier()
    group.close()

    # ---- training: forward + backward across the group == the single-rank pass on the whole problem,
    # with rows pushed to [token * topk + slot] and with rows pushed into receive streams
    whole = mok.Shape("whole", E, H, I, shape.topk, shape.tokens * world)
    single = mok.MoKHost(whole, device=dev)
    single.load_weights(wg * 2.5, wu * 2.5, wd * 2.5, train=True)
    L = shape.tokens
    eq = lambda a, b: torch.equal(a.contiguous().view(torch.int16 if a.dtype == torch.bfloat16 else torch.int32),
                                  b.contiguous().view(torch.int16 if b.dtype == torch.bfloat16 else torch.int32))
    for stream in (False, True):
        group = ep.IpcGroup(shape, rank, world, dev, train=True, stream=stream)
        host = ep.EpMoKHost(shape, rank, group)
        host.load_weights(wg[rank * El:(rank + 1) * El] * 2.5, wu[rank * El:(rank + 1) * El] * 2.5, wd[rank * El:(rank + 1) * El] * 2.5, train=True)
        for generation in (1, 3):
            inputs = [mok.MoKHost.new_inputs(shape, generation, dev, rank=r, world=world) for r in range(world)]
            gen = torch.Generator(device=dev).manual_seed(77 + generation)
            d_outs = [torch.randn(L, H, generator=gen, device=dev).to(torch.bfloat16) for _ in range(world)]
            joined = mok.Inputs(torch.cat([i.x for i in inputs]), torch.cat([i.experts for i in inputs]), torch.cat([i.router for i in inputs]))
            out_single = single.forward(joined, train=True)["output"].clone()
            want = {k: v.clone() for k, v in single.backward(torch.cat(d_outs)).items()}
            host.buffers["d_x_routed_buffer"].fill_(float("nan"))
            out = host.forward(inputs[rank], train=True)["output"]
            g = host.backward(d_outs[rank])
            torch.cuda.synchronize()
            tag = (rank, generation, "streams" if stream else "slots")
            assert eq(out, out_single[rank * L:(rank + 1) * L]), (tag, "output")
            assert torch.isfinite(g["d_x"].float()).all()
            assert eq(g["d_x"], want["d_x"][rank * L:(rank + 1) * L]), (tag, "d_x")
            assert eq(g["d_router_weights"], want["d_router_weights"][rank * L:(rank + 1) * L]), (tag, "d_router_weights")
            for name in ("d_w_routed_gate", "d_w_routed_up", "d_w_routed_down"):
                assert eq(g[name], want[name][rank * El:(rank + 1) * El]), (tag, name)
        torch.cuda.synchronize()
        dist.barrier()
        group.close()
    # ---- the bf16 routed precision: forward + backward across the group == the single-rank bf16 pass
    single_bf = mok.MoKHost(whole, device=dev, precision="bf16")
    single_bf.load_weights(wg * 2.5, wu * 2.5, wd * 2.5, train=True)
    group = ep.IpcGroup(shape, rank, world, dev, train=True)
    host = ep.EpMoKHost(shape, rank, group, precision="bf16")
    host.load_weights(wg[rank * El:(rank + 1) * El] * 2.5, wu[rank * El:(rank + 1) * El] * 2.5, wd[rank * El:(rank + 1) * El] * 2.5, train=True)
    for generation in (1, 3):
        inputs = [mok.MoKHost.new_inputs(shape, generation, dev, rank=r, world=world) for r in range(world)]
        gen = torch.Generator(device=dev).manual_seed(177 + generation)
        d_outs = [torch.randn(L, H, generator=gen, device=dev).to(torch.bfloat16) for _ in range(world)]
        joined = mok.Inputs(torch.cat([i.x for i in inputs]), torch.cat([i.experts for i in inputs]), torch.cat([i.router for i in inputs]))
        out_single = single_bf.forward(joined, train=True)["output"].clone()
        want = {k: v.clone() for k, v in single_bf.backward(torch.cat(d_outs)).items()}
        host.buffers["d_x_routed_buffer"].fill_(float("nan"))
        out = host.forward(inputs[rank], train=True)["output"]
        g = host.backward(d_outs[rank])
        torch.cuda.synchronize()
        tag = (rank, generation, "bf16")
        assert eq(out, out_single[rank * L:(rank + 1) * L]), (tag, "output")
        assert torch.isfinite(g["d_x"].float()).all()
        assert eq(g["d_x"], want["d_x"][rank * L:(rank + 1) * L]), (tag, "d_x")
        assert eq(g["d_router_weights"], want["d_router_weights"][rank * L:(rank + 1) * L]), (tag, "d_router_weights")
        for name in ("d_w_routed_gate", "d_w_routed_up", "d_w_routed_down"):
            assert eq(g[name], want[name][rank * El:(rank + 1) * El]), (tag, name)
    torch.cuda.synchronize()
    dist.barrier()
    group.close()
    dist.destroy_process_group()
    if rank == 0:
        print("EP CHILD OK")


if __name__ == "__main__":
    main()
