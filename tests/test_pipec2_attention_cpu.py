"""The prefill attention kernel's owners through the link driver, without a GPU: seven packages, three
compositions, the solved map (K/V ring depth 2, S / P / O in 512 tensor-memory columns, the softmax
owner on a warpgroup boundary), arrivals from a subset of a role's warps, and the solve staying
fast with fifteen claims in shared memory."""
import copy
import time

import pytest

from pipelink_b200.pipec2 import contracts, link as linker, schema
from pipelink_b200.pipec2.model import PipeLinkError
from pipelink_b200.stages.attention import build as ab


def _stages(comp="prefill"):
    return [copy.deepcopy(ab.manifests()[m]) for m in ab.COMPOSITIONS[comp]]


def test_owners_and_channels():
    for m in ab.manifests().values():
        schema.validate_manifest(copy.deepcopy(m))
    assert {m["stage"]["id"] for m in ab.manifests().values()} == {
        "attn.load", "attn.load.counters", "attn.mma", "attn.gather.none", "attn.gather.push", "attn.softmax", "attn.softmax.softcap"}
    ms = _stages()
    ch = contracts.pair_channels(ms)
    assert sorted(ch) == ["k_tiles", "output", "q_tiles", "scores", "v_tiles"]
    contracts.check_compatibility(ch)
    exp = {e["channel"]: e for e in contracts.expand_protocols(ch, ms, 1)}
    assert exp["q_tiles"]["full"]["tx_bytes"] == 65536 and exp["k_tiles"]["full"]["tx_bytes"] == 32768
    # four of the softmax owner's eight warps arrive on a head's slot: 128 threads
    assert exp["scores"]["empty"] == {"slots": "pipelink_attn_p_full", "count": 128, "by": "softmax", "tx_bytes": 0}
    bad = _stages()
    for m in bad[1::2]:                       # mma and softmax state the scores channel
        for ep in m["endpoints"]:
            if ep["name"] == "scores":
                ep["protocol"]["empty"]["arrive"]["count"] = 96 + 1      # not a whole number of warps or lanes
    with pytest.raises(PipeLinkError) as err:
        contracts.expand_protocols(contracts.pair_channels(bad), bad, 1)
    assert err.value.failures[0].path == "channels.scores.protocol.empty.arrive.count"


@pytest.mark.parametrize("comp", sorted(ab.COMPOSITIONS))
def test_compositions_solve_quickly_to_the_same_map(comp):
    t0 = time.time()
    fe = linker.front_end(_stages(comp), ab.pipeline_spec(comp, [])["pipeline"])
    assert time.time() - t0 < 20
    b = {k: v[0] for k, v in fe["bindings"].items()}
    assert b["pipelink_attn_kv_depth"] == 2
    assert sorted((b["pipelink_attn_s"], b["pipelink_attn_o"])) == [0, 256]
    assert b["pipelink_attn_warp_softmax"] % 4 == 0
    assert {b["pipelink_attn_q"], b["pipelink_attn_k"], b["pipelink_attn_v"]} == {0, 65536, 131072}
    assert fe["solver"]["high_water"]["smem"] <= 232448 and fe["solver"]["high_water"]["tmem"] == 512


def test_three_k_v_stages_do_not_fit():
    spec = ab.pipeline_spec("prefill", [], values=(3,))["pipeline"]
    with pytest.raises(PipeLinkError) as err:
        linker.front_end(_stages(), spec)
    assert {f.clause_id for f in err.value.failures} <= {"L-BUDGET", "L-OVERLAP"}
