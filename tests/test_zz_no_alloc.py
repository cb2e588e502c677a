"""The schedule entry point for callers that cannot allocate (a plugin that only gets input and
output pointers, a stage behind a broker that owns all workspaces, a serving loop that must not
stall the device with cudaMalloc) keeps its chunk counts in a static device array inside the
library. It must give exactly what the scratch-taking entry point gives, call after call, even
though the array still holds the previous call's counts.

Collected last on purpose: a run that stops at the first failure has then already run every
other test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

FIELDS = ("peer_rank", "peer_token_idx", "dest_row", "num_tokens", "tokens_per_expert", "expert_offsets",
          "block_expert")


def _schedule(mok, _lib, routes, rank, E, padding, noalloc):
    world, tokens, topk = routes.shape
    cap = mok.schedule_capacity(world * tokens * topk, E, padding)
    s = mok.Schedule(world, tokens, topk, E, cap, "cuda")
    st = mok.DeviceStatus("cuda")
    for t in (s.peer_rank, s.peer_token_idx, s.dest_row, s.block_expert):
        t.fill_(-5)
    r = torch.from_numpy(routes.astype(np.int32)).cuda()
    head = (r.data_ptr(), world, tokens, topk, rank * E, E, cap, padding, s.peer_rank.data_ptr(),
            s.peer_token_idx.data_ptr(), s.dest_row.data_ptr(), s.num_tokens.data_ptr(),
            s.tokens_per_expert.data_ptr(), s.expert_offsets.data_ptr(), s.block_expert.data_ptr())
    if noalloc:
        _lib.call("plb_moe_schedule_noalloc", *head, st.buf.data_ptr(), None)
    else:
        _lib.call("plb_moe_schedule", *head, s.scratch.data_ptr(), s.scratch.numel() * 4, st.buf.data_ptr(), None)
    torch.cuda.synchronize()
    st.check()
    return {f: getattr(s, f).cpu().numpy() for f in FIELDS}


def test_noalloc_schedule_matches_on_two_calls_in_a_row(native_lib):
    from pipelink_b200 import _lib, mok
    rng = np.random.default_rng(11)
    # two different problems back to back: the second runs over the first one's leftovers
    cases = [(2, 700, 4, 16, 128), (1, 1500, 2, 8, 256)]
    for world, tokens, topk, experts, padding in cases:
        routes = np.stack([np.stack([rng.permutation(experts)[:topk] for _ in range(tokens)])
                           for _ in range(world)])
        E = experts // world
        for rank in range(world):
            want = _schedule(mok, _lib, routes, rank, E, padding, noalloc=False)
            got = _schedule(mok, _lib, routes, rank, E, padding, noalloc=True)
            for f in FIELDS:
                assert np.array_equal(got[f], want[f]), (f, world, tokens, rank)


def test_noalloc_schedule_rejects_oversized_problems(native_lib):
    from pipelink_b200 import _lib
    limit = native_lib.plb_moe_schedule_noalloc_max_scratch_bytes()
    assert limit == 1 << 20
    # 8 ranks x 65536 tokens x top-8 over 512 local experts needs 8 MiB of counts
    assert native_lib.plb_moe_schedule_scratch_bytes(8, 65536, 8, 512) > limit
    dummy = torch.zeros(64, dtype=torch.int32, device="cuda")
    p = dummy.data_ptr()
    with pytest.raises(_lib.PlbError) as e:
        _lib.call("plb_moe_schedule_noalloc", p, 8, 65536, 8, 0, 512, 128 * 40000, 128, p, p, p, p, p, p, p, p, None)
    assert e.value.code == 2 and "capacity" in str(e.value)
