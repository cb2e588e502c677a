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


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ipc_group_forward_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29531", str(ROOT / "tests" / "ep_child.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "EP CHILD OK" in out.stdout
