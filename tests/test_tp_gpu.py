"""AllGather -> GEMM and GEMM -> ReduceScatter (the reference's examples/comm-overlap compositions).
On one GPU the ranks are emulated in one process; with two GPUs a torchrun child runs the IPC group."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _rel(ref, got):
    return float((got.double() - ref.double()).norm() / ref.double().norm())


def _case(m, n, k, world, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn(m, k, generator=g, device="cuda").to(torch.bfloat16)
    b = (torch.randn(n, k, generator=g, device="cuda") * 0.1).to(torch.bfloat16)
    return a, b, (a.float() @ b.float().T)


@pytest.mark.parametrize("world,m,n,k", [(2, 1024, 1024, 512), (4, 2048, 1024, 1024)])
def test_allgather_gemm_emulated_ranks(native_lib, world, m, n, k):
    from pipelink_b200 import tp
    group = tp.LocalTpGroup(m, n, k, world)
    try:
        ms, nl = m // world, n // world
        for step in range(3):                       # both parities of the gathered buffers, then reuse
            a, b, ref = _case(m, n, k, world, 10 + step)
            outs = group.ag([a[r * ms:(r + 1) * ms] for r in range(world)],
                            [b[r * nl:(r + 1) * nl].contiguous() for r in range(world)])
            torch.cuda.synchronize()
            for r in range(world):
                want = ref[:, r * nl:(r + 1) * nl]
                # one bf16 rounding of an fp32 sum: the only difference is summation order
                assert _rel(want, outs[r]) < 3e-3, (step, r)
                assert torch.equal(outs[r], outs[r].clone())
            # all ranks multiplied the same gathered rows: column blocks of one product
            full = torch.cat(outs, dim=1)
            assert _rel(ref, full) < 3e-3
    finally:
        group.close()


@pytest.mark.parametrize("world,m,n,k", [(2, 1024, 1024, 512), (4, 2048, 1024, 1024)])
def test_gemm_reduce_scatter_emulated_ranks(native_lib, world, m, n, k):
    from pipelink_b200 import tp
    group = tp.LocalTpGroup(m, n, k, world)
    try:
        ms, kl = m // world, k // world
        for step in range(3):
            a, b, ref = _case(m, n, k, world, 20 + step)
            for r in group.ranks:
                r.slots[r.rs_generation & 1].fill_(float("nan"))       # every slot row must be pushed by its source
            a_l = [a[:, r * kl:(r + 1) * kl].contiguous() for r in range(world)]
            b_l = [b[:, r * kl:(r + 1) * kl].contiguous() for r in range(world)]
            outs = [o.clone() for o in group.rs(a_l, b_l)]
            torch.cuda.synchronize()
            # the device sums bf16-rounded partials in rank order: reproduce exactly that
            parts = [(a_l[q].float() @ b_l[q].float().T) for q in range(world)]
            for r in range(world):
                rows = slice(r * ms, (r + 1) * ms)
                assert torch.isfinite(outs[r].float()).all()
                assert _rel(ref[rows], outs[r]) < 1e-2, (step, r)          # bf16 partials: W roundings
                acc = torch.zeros(ms, n, device="cuda")
                for q in range(world):
                    acc = acc + parts[q][rows].to(torch.bfloat16).float()
                assert _rel(acc, outs[r]) < 4e-3, (step, r)
            again = [o.clone() for o in group.rs(a_l, b_l)]                 # other parity, same operands
            for r in range(world):
                assert torch.equal(again[r].view(torch.int16), outs[r].view(torch.int16))    # bitwise repeatable
    finally:
        group.close()


@pytest.mark.parametrize("order", ["ag,ag,rs,ag,ag", "rs,ag,ag", "ag,rs,rs,ag,rs,ag,ag,ag"])
def test_interleaved_ag_and_rs_keep_their_own_generations(native_lib, order):
    """The gathered buffers follow the number of ag steps and the receive slots the number of rs steps:
    any interleaving gives correct results and a clean status (a shared step counter made the
    all-gather GEMM wait for a counter value that its parity never reaches)."""
    from pipelink_b200 import tp
    world, m, n, k = 2, 1024, 1024, 512
    group = tp.LocalTpGroup(m, n, k, world)
    try:
        ms, nl, kl = m // world, n // world, k // world
        for step, op in enumerate(order.split(",")):
            a, b, ref = _case(m, n, k, world, 40 + step)
            if op == "ag":
                outs = group.ag([a[r * ms:(r + 1) * ms] for r in range(world)],
                                [b[r * nl:(r + 1) * nl].contiguous() for r in range(world)])
                torch.cuda.synchronize()
                assert _rel(ref, torch.cat(outs, dim=1)) < 3e-3, (step, op)
            else:
                for r in group.ranks:
                    r.slots[r.rs_generation & 1].fill_(float("nan"))
                outs = group.rs([a[:, r * kl:(r + 1) * kl].contiguous() for r in range(world)],
                                [b[:, r * kl:(r + 1) * kl].contiguous() for r in range(world)])
                torch.cuda.synchronize()
                assert _rel(ref, torch.cat(outs, dim=0)) < 1e-2, (step, op)
    finally:
        group.close()


def test_allgather_gemm_reports_rows_that_never_arrive(native_lib):
    """A readiness counter nobody advances: the load lane's wait runs out (about a second), the kernel
    records status 5 and returns; the context stays usable."""
    from pipelink_b200 import tp
    group = tp.LocalTpGroup(512, 512, 256, 2)
    try:
        r0 = group.ranks[0]
        b = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
        r0.ag_gemm(b)                               # no push was issued
        with pytest.raises(RuntimeError, match="status 5"):
            r0.status.check("unpushed rows")
        r0.status.reset()
        a, bb, ref = _case(512, 512, 256, 2, 3)
        outs = group.ag([a[:256], a[256:]], [bb[:256].contiguous(), bb[256:].contiguous()])
        assert _rel(ref[:, :256], outs[0]) < 3e-3
    finally:
        group.close()


@pytest.mark.parametrize("world", [2, 4])
def test_ipc_tp_group_real_gpus(world):
    from tests.ranks import gpu_count, run_ranks
    if gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_ranks("tp_child.py", world, 29551 + world, "TP CHILD OK")
