"""GPU parity for causal prefill attention (tcgen05) and its context-parallel composition.

Inputs are the reference's Philox fixtures (U[-2,2) rounded to bf16); the oracle evaluates full
visible keys for sampled rows (all rows for short sequences); the predicate is the reference's
``|a - r| <= 0.02 + 0.02 |r|`` for O and LSE. Context parallel runs W ranks in one process on one
GPU (all pushes, then each rank's attention) and must reproduce the single-GPU result bitwise."""
import numpy as np
import pytest
import torch

from oracle import attention as oa

pytestmark = pytest.mark.gpu


def _inputs(S, Hq, Hkv, case=0):
    q = oa.philox_bf16(S * Hq * 128, case, 1).reshape(S, Hq, 128)
    k = oa.philox_bf16(S * Hkv * 128, case, 2).reshape(S, Hkv, 128)
    v = oa.philox_bf16(S * Hkv * 128, case, 3).reshape(S, Hkv, 128)
    dev = lambda a: torch.from_numpy(a).to(torch.bfloat16).cuda()
    return (q, k, v), (dev(q), dev(k), dev(v))


@pytest.mark.parametrize("S,Hq,Hkv,rows", [(128, 1, 1, None), (256, 4, 1, None), (512, 8, 2, None), (1024, 4, 4, "boundary"),
                                           (4096, 8, 2, "boundary")])
def test_attention_vs_oracle(native_lib, S, Hq, Hkv, rows):
    from pipelink_b200 import attention as att
    (q, k, v), (dq, dk, dv) = _inputs(S, Hq, Hkv, case=S)
    out, lse = att.attention_fwd(dq[None], dk[None], dv[None])
    torch.cuda.synchronize()
    sel = list(range(S)) if rows is None else oa.boundary_rows(S, extra=(S // 2 + 3, S - 130))
    ref_o, ref_lse = oa.reference_rows(q, k, v, sel, 1.0 / np.sqrt(128.0))
    got_o = out[0].float().cpu().numpy()[sel]
    got_lse = lse.cpu().numpy()[:, sel]
    assert np.isfinite(got_o).all()
    assert oa.matches(got_o, ref_o) == 0, np.abs(got_o - ref_o).max()
    assert oa.matches(got_lse, ref_lse) == 0, np.abs(got_lse - ref_lse).max()


@pytest.mark.parametrize("pair", [False, True])
def test_attention_growing_scores_both_kernels(native_lib, pair):
    """Keys grow with position, so the row maximum keeps rising by more than the two-head kernel's
    rescale threshold: its deferred rescale of O in TMEM has to fire in late blocks; the one-head
    kernel on the same inputs is the cross-check."""
    from pipelink_b200 import attention as att
    S, Hq, Hkv = 2048, 4, 2
    (q, k, v), _ = _inputs(S, Hq, Hkv, case=11)
    ramp = (1.0 + 5.0 * np.arange(S, dtype=np.float32) / S)[:, None, None]
    k = torch.from_numpy(k * ramp).to(torch.bfloat16).float().numpy()
    dev = lambda a: torch.from_numpy(a).to(torch.bfloat16).cuda()
    out, lse = att.attention_fwd(dev(q)[None], dev(k)[None], dev(v)[None], pair_heads=pair)
    torch.cuda.synchronize()
    sel = oa.boundary_rows(S, extra=(S // 2 + 3, S - 130, 700, 1300))
    ref_o, ref_lse = oa.reference_rows(q, k, v, sel, 1.0 / np.sqrt(128.0))
    got_o = out[0].float().cpu().numpy()[sel]
    got_lse = lse.cpu().numpy()[:, sel]
    assert np.isfinite(got_o).all()
    assert oa.matches(got_o, ref_o) == 0, np.abs(got_o - ref_o).max()
    assert oa.matches(got_lse, ref_lse) == 0, np.abs(got_lse - ref_lse).max()


@pytest.mark.parametrize("Hq,Hkv,window,softcap", [(4, 2, 200, 0.0), (4, 2, 128, 0.0), (4, 4, 1000, 0.0), (4, 2, 0, 30.0),
                                                    (2, 2, 0, 8.0), (8, 2, 300, 20.0)])
def test_window_and_softcap_variants_vs_oracle(native_lib, Hq, Hkv, window, softcap):
    """The reference's mask-window and score-softcap stage variants on both kernels (two heads per
    CTA when Hq / Hkv is even, one otherwise): rows around every block and window edge."""
    from pipelink_b200 import attention as att
    S = 1536
    (q, k, v), (dq, dk, dv) = _inputs(S, Hq, Hkv, case=window + int(softcap))
    out, lse = att.attention_fwd(dq[None], dk[None], dv[None], window=window, softcap=softcap)
    torch.cuda.synchronize()
    extra = [S // 2 + 3, S - 130]
    if window:
        extra += [window - 1, window, window + 1, 2 * window + 5, 127 + window, 128 + window, S - 1]
    sel = sorted({r for r in oa.boundary_rows(S, extra=tuple(e for e in extra if 0 <= e < S))})
    ref_o, ref_lse = oa.reference_rows(q, k, v, sel, 1.0 / np.sqrt(128.0), window=window, softcap=softcap)
    got_o = out[0].float().cpu().numpy()[sel]
    got_lse = lse.cpu().numpy()[:, sel]
    assert np.isfinite(got_o).all()
    assert oa.matches(got_o, ref_o) == 0, np.abs(got_o - ref_o).max()
    assert oa.matches(got_lse, ref_lse) == 0, np.abs(got_lse - ref_lse).max()


def test_attention_deterministic(native_lib):
    from pipelink_b200 import attention as att
    _, (dq, dk, dv) = _inputs(1024, 8, 2, case=7)
    a, la = att.attention_fwd(dq[None], dk[None], dv[None])
    b, lb = att.attention_fwd(dq[None], dk[None], dv[None])
    assert torch.equal(a.view(torch.int16), b.view(torch.int16)) and torch.equal(la, lb)


@pytest.mark.parametrize("world,S", [(2, 1024), (4, 2048)])
def test_context_parallel_matches_single_gpu(native_lib, world, S):
    from pipelink_b200 import attention as att, ep
    Hq, Hkv = 8, 2
    (q, k, v), (dq, dk, dv) = _inputs(S, Hq, Hkv, case=world)
    full_o, full_lse = att.attention_fwd(dq[None], dk[None], dv[None])
    torch.cuda.synchronize()
    layout = att.CpRank.slab_layout(S, Hkv)
    slabs = [ep.sym_alloc(layout["nbytes"]) for _ in range(world)]
    try:
        ranks = [att.CpRank(S, Hq, Hkv, r, world, slabs, layout, "cuda") for r in range(world)]
        for rnk in ranks:   # poison the gathered buffers: a block that was not pushed cannot look right
            rnk.k_gather.fill_(float("nan"))
            rnk.v_gather.fill_(float("nan"))
        for step in range(2):   # two steps: counters advance by one per step and are never reset
            for r, rnk in enumerate(ranks):
                rnk.push(att.shard_zigzag(dk, world, r), att.shard_zigzag(dv, world, r))
            for r, rnk in enumerate(ranks):
                o, lse = rnk.attend(att.shard_zigzag(dq, world, r))
                torch.cuda.synchronize()
                rnk.status.check(f"cp rank {r}")
                pos = torch.from_numpy(oa.zigzag_rows(S, world, r)).cuda()
                assert torch.equal(o.view(torch.int16), full_o[0][pos].view(torch.int16)), (world, r, step)
                assert torch.equal(lse, full_lse[:, pos])
                assert (rnk.ready.cpu().numpy()[: (2 * world - r) * (S // (2 * world)) // 128] == step + 1).all()
    finally:
        torch.cuda.synchronize()
        from pipelink_b200 import _lib
        for p in slabs:
            _lib.call("plb_sym_free", p)


@pytest.mark.parametrize("S,Hq,Hkv", [(2048, 8, 2), (8192, 8, 4)])
def test_kv_exchange_inside_the_attention_launch_single_rank(native_lib, S, Hq, Hkv):
    """The gather warps of the attention kernel on a group of one: every K/V block this rank owns goes
    from its local tensors into its own gathered buffers in pieces, counted per block, while the same
    launch's load lanes wait for those counts. All CTAs of the launch are resident at once and the
    gather warps wait for nothing, so one GPU can run it (ranks emulated as separate launches could
    not: an earlier launch would wait for a later one). Result: the plain kernel's, bit for bit."""
    from pipelink_b200 import _lib, attention as att, ep
    (q, k, v), (dq, dk, dv) = _inputs(S, Hq, Hkv, case=3)
    full_o, full_lse = att.attention_fwd(dq[None], dk[None], dv[None])
    torch.cuda.synchronize()
    layout = att.CpRank.slab_layout(S, Hkv)
    slab = ep.sym_alloc(layout["nbytes"])
    try:
        rnk = att.CpRank(S, Hq, Hkv, 0, 1, [slab], layout, "cuda", fused_push=True)
        rnk.k_gather.fill_(float("nan"))
        rnk.v_gather.fill_(float("nan"))
        for step in range(3):
            o, lse = rnk.step(dq, dk, dv, distributed=False)
            torch.cuda.synchronize()
            rnk.status.check(f"fused push, step {step}")
            assert torch.equal(o.view(torch.int16), full_o[0].view(torch.int16)), step
            assert torch.equal(lse, full_lse), step
            assert (rnk.ready.cpu().numpy() == (step + 1) * att.CpRank.PARTS).all()
    finally:
        torch.cuda.synchronize()
        _lib.call("plb_sym_free", slab)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_context_parallel_real_gpus(world):
    from tests.ranks import gpu_count, run_ranks
    if gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    run_ranks("cp_child.py", world, 29561 + world, "CP CHILD OK")



def test_attention_seq32768_boundary_rows(native_lib):
    """The benchmarked prefill size (S = 32768, 32 query / 8 KV heads, d = 128, N(0,1) inputs as the
    configuration names them): boundary and interior spot rows against the fp64 oracle over all
    visible keys (campaigns/attention/src/slot/family.cuh:156-229), the reference's predicate."""
    from pipelink_b200 import attention as att
    S, Hq, Hkv = 32768, 32, 8
    g = torch.Generator(device="cuda").manual_seed(0)
    q = torch.randn(1, S, Hq, 128, generator=g, device="cuda").to(torch.bfloat16)
    k = torch.randn(1, S, Hkv, 128, generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn(1, S, Hkv, 128, generator=g, device="cuda").to(torch.bfloat16)
    out, lse = att.attention_fwd(q, k, v)
    torch.cuda.synchronize()
    sel = [0, 1, 127, 128, 129, 4095, 4096, 16383, 16384, 16385, 20001, S - 130, S - 129, S - 128, S - 2, S - 1]
    idx = torch.tensor(sel, device="cuda")
    q_rows = q[0, idx].float().cpu().numpy()                   # only the sampled query rows travel to the host
    kf, vf = k[0].float().cpu().numpy(), v[0].float().cpu().numpy()
    ref_o, ref_lse = oa.reference_rows(q_rows, kf, vf, list(range(len(sel))), 1.0 / np.sqrt(128.0), q_pos=sel)
    got_o = out[0, idx].float().cpu().numpy()
    got_lse = lse[:, idx].cpu().numpy()
    assert np.isfinite(got_o).all()
    assert oa.matches(got_o, ref_o) == 0, np.abs(got_o - ref_o).max()
    assert oa.matches(got_lse, ref_lse) == 0, np.abs(got_lse - ref_lse).max()
