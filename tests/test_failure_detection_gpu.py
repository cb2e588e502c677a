"""Failure detection on the device: every wait in these kernels has a limit of about a second,
after which the kernel records where it gave up in the caller's status record, lets its other
waits give up too, and returns. Each test makes one wait run out by leaving a flag or counter
that nothing sets, reads the status on the host, and then runs the same kernel normally to show
the context is still usable. Nothing here faults, traps or hangs the GPU."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TIMEOUT_COUNTER = 5     # ST_TIMEOUT_COUNTER: a readiness counter never reached its target


def _status_fields(status):
    vals = status.buf.cpu().tolist()
    return dict(code=vals[0], cta=vals[1], what=vals[2], observed=vals[3] & 0xFFFFFFFF, expected=vals[4] & 0xFFFFFFFF)


def test_group_barrier_reports_the_peer_that_never_arrived(native_lib):
    """Rank 0 of a two-rank group enters the flag barrier alone: its wait for rank 1's arrival runs
    out and names the peer (what = 200 + peer)."""
    from pipelink_b200 import _lib, ep, mok
    slabs = [ep.sym_alloc(4096) for _ in range(2)]
    try:
        flags = torch.tensor(slabs, dtype=torch.int64, device="cuda")
        state = torch.zeros(1, dtype=torch.int32, device="cuda")
        status = mok.DeviceStatus("cuda")
        _lib.call("plb_ep_barrier", flags.data_ptr(), state.data_ptr(), 0, 2, status.buf.data_ptr(), mok._stream())
        torch.cuda.synchronize()
        f = _status_fields(status)
        assert (f["code"], f["what"], f["observed"], f["expected"]) == (TIMEOUT_COUNTER, 201, 0, 1), f
        with pytest.raises(RuntimeError, match="readiness-counter timeout"):
            status.check("barrier")
        assert int(state.item()) == 1, "the generation advances even after a failure"
        # the context is usable: the next barrier (generation 2) passes once rank 1's arrival is there;
        # the host plays rank 1 by writing the flag, so no two kernels wait on each other
        status.reset()
        ep.tensor_from_ptr(slabs[0], (64,), torch.int32, torch.device("cuda"))[1] = 2
        _lib.call("plb_ep_barrier", flags.data_ptr(), state.data_ptr(), 0, 2, status.buf.data_ptr(), mok._stream())
        torch.cuda.synchronize()
        status.check("barrier after recovery")
        assert int(state.item()) == 2
    finally:
        torch.cuda.synchronize()
        for p in slabs:
            _lib.call("plb_sym_free", p)


def test_context_parallel_attention_reports_the_block_that_was_never_published(native_lib):
    """The attention load lane acquires a per-block readiness counter before its first TMA of a
    remote block. With counters that nothing bumps the wait runs out, every role of every CTA
    leaves, and the status names the counter wait (what = 300)."""
    from oracle import attention as oa
    from pipelink_b200 import attention as att, mok
    S, Hq, Hkv = 512, 4, 2
    dev = lambda a: torch.from_numpy(a).to(torch.bfloat16).cuda()
    q = dev(oa.philox_bf16(S * Hq * 128, 3, 1).reshape(S, Hq, 128))
    k = dev(oa.philox_bf16(S * Hkv * 128, 3, 2).reshape(S, Hkv, 128))
    v = dev(oa.philox_bf16(S * Hkv * 128, 3, 3).reshape(S, Hkv, 128))
    out = torch.zeros_like(q)
    lse = torch.zeros((Hq, S), dtype=torch.float32, device="cuda")
    step = att.heads_per_work(Hq, Hkv)
    work = torch.from_numpy(att.causal_work(1, S, Hq, step)).cuda()
    ready = torch.zeros(S // 128, dtype=torch.int32, device="cuda")     # never published
    status = mok.DeviceStatus("cuda")
    att._launch(q, k, v, out, lse, work, step, S, ready, 1, status)
    torch.cuda.synchronize()
    f = _status_fields(status)
    assert (f["code"], f["what"], f["observed"], f["expected"]) == (TIMEOUT_COUNTER, 300, 0, 1), f
    # the same launch with the blocks published completes and matches the plain kernel
    ready.fill_(1)
    status.reset()
    att._launch(q, k, v, out, lse, work, step, S, ready, 1, status)
    torch.cuda.synchronize()
    status.check("attention after recovery")
    want, want_lse = att.attention_fwd(q[None], k[None], v[None])
    assert torch.equal(out.view(torch.int16), want[0].view(torch.int16)) and torch.equal(lse, want_lse)


def test_decode_reports_the_dependency_that_was_never_signalled(native_lib):
    """One instruction of the decode stream waits on a counter nothing bumps: the consumers'
    bounded wait records (opcode * 100 + layer), the producer warp and every other CTA leave."""
    from pipelink_b200 import decode as hd
    torch.manual_seed(0)
    L, V = 1, 1024
    mk = lambda *s: (torch.randn(*s, device="cuda") * 0.02).to(torch.bfloat16)
    ones = lambda *s: torch.ones(*s, device="cuda", dtype=torch.bfloat16)
    w = dict(qkv_w=mk(L, hd.QKV_ROWS, hd.HIDDEN), o_w=mk(L, hd.HIDDEN, hd.HIDDEN), up_w=mk(L, hd.FFN, hd.HIDDEN),
             gate_w=mk(L, hd.FFN, hd.HIDDEN), down_w=mk(L, hd.HIDDEN, hd.FFN), attn_norm=ones(L, hd.HIDDEN),
             mlp_norm=ones(L, hd.HIDDEN), lm_norm=ones(hd.HIDDEN), lm_head=mk(V, hd.HIDDEN))
    s = hd.DecodeSession(w, max_seq_len=16, partitions=1)
    s.start(1, 0)
    s.decode(1)                                   # a healthy token first
    good = s.instructions.clone()
    # the O projection (opcode 4) now waits for 1,000,000 arrivals on its counter
    inst = good.clone()
    rows = inst[:, :, 0] == hd.OP_OPROJ
    inst[:, :, 7][rows] = 1_000_000
    s.instructions.copy_(inst)
    s.start(1, 0)
    s.step()
    torch.cuda.synchronize()
    f = _status_fields(s.status)
    assert f["code"] == TIMEOUT_COUNTER and f["what"] == hd.OP_OPROJ * 100 and f["expected"] == 1_000_000, f
    assert f["observed"] == hd.KV_HEADS, "all eight KV heads had signalled; the target was wrong"
    # restore the stream: the session decodes the same token as before the failure
    first = int(s.token_out[1].item())
    s.instructions.copy_(good)
    s.start(1, 0)
    s.decode(1)
    assert int(s.token_out[1].item()) == first
