"""Expert-parallel forward. On one GPU the ranks of a group are emulated inside one process
(all slabs on the same device, phases run rank after rank, no flag barrier launched); with two
or more GPUs a torchrun child job runs the real IPC group and compares with the same oracle."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import moe as omoe

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _f(t):
    return t.detach().float().cpu().numpy()


def make_group_case(mok, shape, world, seed=0):
    torch.manual_seed(seed)
    E, H, I = shape.experts, shape.hidden, shape.intermediate
    wg = (torch.randn(E, I, H, device="cuda") * 0.02).to(torch.bfloat16)
    wu = (torch.randn(E, I, H, device="cuda") * 0.02).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device="cuda") * 0.02).to(torch.bfloat16)
    inputs = [mok.MoKHost.new_inputs(shape, 1 + (r == 1) * 2, "cuda", rank=r, world=world) for r in range(world)]
    return wg, wu, wd, inputs


@pytest.mark.parametrize("world,shape_args", [(2, ("ep2", 8, 512, 256, 2, 256)), (4, ("ep4", 16, 256, 256, 4, 128))])
def test_local_group_forward_vs_oracle(native_lib, world, shape_args):
    from pipelink_b200 import ep, mok
    shape = mok.Shape(*shape_args)
    wg, wu, wd, inputs = make_group_case(mok, shape, world)   # rank 1 gets concentrated routing
    group = ep.LocalGroup(shape, world, "cuda")
    try:
        hosts = [ep.EpMoKHost(shape, r, group) for r in range(world)]
        El = shape.experts // world
        for r, h in enumerate(hosts):
            h.load_weights(wg[r * El:(r + 1) * El], wu[r * El:(r + 1) * El], wd[r * El:(r + 1) * El])
            h.buffers["combine_buffer"].fill_(float("nan"))
        outs = ep.forward_local_group(hosts, inputs)
        torch.cuda.synchronize()
        weights = omoe.quantize_weights(_f(wg), _f(wu), _f(wd))
        ref = omoe.forward_multi_rank([_f(i.x) for i in inputs],
                                      [i.experts.cpu().numpy().astype(np.int32) for i in inputs],
                                      [i.router.cpu().numpy() for i in inputs], weights, world,
                                      padding=mok.expert_padding())
        for r, h in enumerate(hosts):
            sched = ref["schedules"][r]
            total = int(sched["num_tokens"][0])
            assert int(h.schedule.num_tokens.item()) == total
            assert np.array_equal(h.schedule.peer_rank.cpu().numpy()[:total], sched["peer_rank"][:total])
            assert np.array_equal(h.schedule.dest_row.cpu().numpy()[:total], sched["dest_row"][:total])
            # pulled rows are bit-identical to quantising the gathered rows
            xq, xsc = omoe.dispatch([_f(i.x) for i in inputs], sched)
            assert np.array_equal(h.buffers["x_routed_fp8"].cpu().numpy()[:total], xq)
            assert np.array_equal(h.buffers["x_routed_sc"].cpu().numpy()[: total // 128], xsc)
            comb = _f(h.buffers["combine_buffer"])
            assert np.isfinite(comb).all()          # every (token, slot) row was pushed by some rank
            s = omoe.error_stats(ref["combine"][r], comb)
            assert s["relative"] <= 2e-2, s
            assert np.array_equal(_f(outs[r]), omoe.fwd_epilogue(comb, inputs[r].router.cpu().numpy()))
            s = omoe.error_stats(ref["outputs"][r], _f(outs[r]))
            assert s["relative"] <= 2e-2, s
    finally:
        torch.cuda.synchronize()
        group.close()


@pytest.mark.parametrize("stream", [False, True], ids=["slots", "streams"])
@pytest.mark.parametrize("world,shape_args", [(2, ("ep2b", 8, 512, 256, 2, 256)), (4, ("ep4b", 8, 256, 256, 4, 128)),
                                              (4, ("ep4c", 8, 256, 256, 4, 256))])
def test_local_group_backward_equals_the_single_rank_backward(native_lib, world, shape_args, stream):
    """Forward + backward over a group must give, bit for bit, what one rank holding every token and
    every expert computes: an expert's rows arrive in the same order on the rank that owns it, so
    every quantisation block, GEMM and reduction sees the same operands. (The single-rank backward
    is itself held to the CPU oracle in test_moe_backward_gpu.py.)"""
    from pipelink_b200 import ep, mok
    shape = mok.Shape(*shape_args)
    wg, wu, wd, inputs = make_group_case(mok, shape, world, seed=3)
    wg, wu, wd = wg * 2.5, wu * 2.5, wd * 2.5
    torch.manual_seed(11)
    d_outs = [torch.randn(shape.tokens, shape.hidden, device="cuda").to(torch.bfloat16) for _ in range(world)]
    # one rank, all tokens, all experts
    whole = mok.Shape("whole", shape.experts, shape.hidden, shape.intermediate, shape.topk, shape.tokens * world)
    single = mok.MoKHost(whole)
    single.load_weights(wg, wu, wd, train=True)
    joined = mok.Inputs(torch.cat([i.x for i in inputs]), torch.cat([i.experts for i in inputs]), torch.cat([i.router for i in inputs]))
    out_single = single.forward(joined, train=True)["output"].clone()
    want = {k: v.clone() for k, v in single.backward(torch.cat(d_outs)).items()}
    group = ep.LocalGroup(shape, world, "cuda", train=True, stream=stream)
    try:
        hosts = [ep.EpMoKHost(shape, r, group) for r in range(world)]
        El, L = shape.experts // world, shape.tokens
        for r, h in enumerate(hosts):
            h.load_weights(wg[r * El:(r + 1) * El], wu[r * El:(r + 1) * El], wd[r * El:(r + 1) * El], train=True)
            h.buffers["d_x_routed_buffer"].fill_(float("nan"))      # every (token, slot) row must be pushed by some rank
            if stream:      # rows travel through the receive streams instead: the index must reach every one
                h.d_x_recv.fill_(float("nan"))
                h.recv.fill_(float("nan"))
        outs = ep.forward_local_group(hosts, inputs, train=True)
        grads = ep.backward_local_group(hosts, d_outs)
        torch.cuda.synchronize()
        eq = lambda a, b: torch.equal(a.contiguous().view(torch.int16 if a.dtype == torch.bfloat16 else torch.int32),
                                      b.contiguous().view(torch.int16 if b.dtype == torch.bfloat16 else torch.int32))
        for r in range(world):
            assert eq(outs[r], out_single[r * L:(r + 1) * L]), ("output", r)
            g = grads[r]
            assert torch.isfinite(g["d_x"].float()).all()
            assert eq(g["d_x"], want["d_x"][r * L:(r + 1) * L]), ("d_x", r)
            assert eq(g["d_router_weights"], want["d_router_weights"][r * L:(r + 1) * L]), ("d_router_weights", r)
            for name in ("d_w_routed_gate", "d_w_routed_up", "d_w_routed_down"):
                assert eq(g[name], want[name][r * El:(r + 1) * El]), (name, r)
    finally:
        torch.cuda.synchronize()
        group.close()


@pytest.mark.parametrize("world,shape_args", [(2, ("ep2h", 8, 512, 256, 2, 256)), (4, ("ep4h", 8, 256, 256, 4, 128))])
def test_local_group_bf16_precision_equals_the_single_rank_forward(native_lib, world, shape_args):
    """bf16 routed precision over a group: rows are dispatched as bf16 from the home ranks' token
    buffers and pushed back from the down GEMM; the result equals, bit for bit, one rank holding
    every token and expert (itself held to the oracle in test_moe_gpu.py)."""
    from pipelink_b200 import ep, mok
    shape = mok.Shape(*shape_args)
    wg, wu, wd, inputs = make_group_case(mok, shape, world, seed=5)
    whole = mok.Shape("whole", shape.experts, shape.hidden, shape.intermediate, shape.topk, shape.tokens * world)
    single = mok.MoKHost(whole, precision="bf16")
    single.load_weights(wg, wu, wd)
    joined = mok.Inputs(torch.cat([i.x for i in inputs]), torch.cat([i.experts for i in inputs]), torch.cat([i.router for i in inputs]))
    want = single.forward(joined)["output"].clone()
    with pytest.raises(ValueError):
        plain = ep.LocalGroup(shape, world, "cuda")
        try:
            ep.EpMoKHost(shape, 0, plain, precision="bf16")        # no peer-visible bf16 tokens in this slab
        finally:
            plain.close()
    group = ep.LocalGroup(shape, world, "cuda", train=True)
    try:
        hosts = [ep.EpMoKHost(shape, r, group, precision="bf16") for r in range(world)]
        El, L = shape.experts // world, shape.tokens
        for r, h in enumerate(hosts):
            h.load_weights(wg[r * El:(r + 1) * El], wu[r * El:(r + 1) * El], wd[r * El:(r + 1) * El])
            h.buffers["combine_buffer"].fill_(float("nan"))
        outs = ep.forward_local_group(hosts, inputs)
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.isfinite(outs[r].float()).all()
            assert torch.equal(outs[r].view(torch.int16), want[r * L:(r + 1) * L].view(torch.int16)), r
    finally:
        torch.cuda.synchronize()
        group.close()


@pytest.mark.parametrize("world,shape_args", [(2, ("ep2s", 8, 512, 256, 2, 256)), (4, ("ep4s", 16, 256, 256, 4, 384)),
                                              (2, ("ep2f", 8, 512, 256, 2, 512)), (4, ("ep4f", 16, 256, 256, 4, 512))])
def test_local_group_receive_streams_equal_the_slot_layout(native_lib, world, shape_args):
    """The combine push into per-source receive streams plus the indexed epilogue gives the same
    output, bit for bit, as the push into [token * topk + slot]; every stream position is used once.
    Where tokens * topk is a multiple of 1024 the schedule launches write the stream positions
    themselves (the last two cases): they must be the positions the separate pass computes."""
    from pipelink_b200 import ep, mok
    shape = mok.Shape(*shape_args)
    wg, wu, wd, inputs = make_group_case(mok, shape, world, seed=7)
    El = shape.experts // world
    outs = {}
    for stream in (False, True):
        group = ep.LocalGroup(shape, world, "cuda", stream=stream)
        try:
            hosts = [ep.EpMoKHost(shape, r, group) for r in range(world)]
            for r, h in enumerate(hosts):
                h.load_weights(wg[r * El:(r + 1) * El], wu[r * El:(r + 1) * El], wd[r * El:(r + 1) * El])
                assert h.stream_push == stream
                if stream:
                    h.recv_index.fill_(-7)
            for step in range(2):           # second step: different routing, positions recomputed
                res = ep.forward_local_group(hosts, [mok.MoKHost.new_inputs(shape, 1 + step + (r == 1) * 2, "cuda", rank=r, world=world)
                                                     for r in range(world)])
                outs[(stream, step)] = [o.clone() for o in res]
            torch.cuda.synchronize()
            if stream:
                Lk = shape.tokens * shape.topk
                for h in hosts:
                    idx = h.recv_index.cpu().numpy()
                    assert (idx >= 0).all() and (idx < world * Lk).all()       # every (token, slot) was indexed
                    assert len(np.unique(idx)) == Lk
                assert hosts[0].schedule_writes_streams == (Lk % 1024 == 0)
                if hosts[0].schedule_writes_streams:
                    folded = [(h.stream_row.clone(), h.recv_index.clone()) for h in hosts]
                    for h in hosts:
                        h.stream_row.fill_(-9)
                        h.recv_index.fill_(-9)
                    for h in hosts:
                        h.stream_rows()                 # the separate pass, on the same schedule
                    torch.cuda.synchronize()
                    for h, (rows, index) in zip(hosts, folded):
                        total = int(h.schedule.num_tokens.item())
                        assert torch.equal(rows[:total], h.stream_row[:total])
                        assert torch.equal(index, h.recv_index)
        finally:
            torch.cuda.synchronize()
            group.close()
    for step in range(2):
        for r in range(world):
            assert torch.equal(outs[(True, step)][r].view(torch.int16), outs[(False, step)][r].view(torch.int16)), (step, r)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ipc_group_forward_and_backward_real_gpus(world):
    """One process per GPU over CUDA IPC (tests/ep_child.py): forward vs the oracle, host pipeline,
    in-kernel dispatch, receive streams, and forward + backward bitwise against the single-rank pass."""
    from tests.ranks import gpu_count, run_ranks
    if gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_ranks("ep_child.py", world, 29531 + world, "EP CHILD OK")
