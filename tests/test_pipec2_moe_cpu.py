"""The link driver on the MoE grouped-GEMM packages, without a GPU: CTA-pair topology, cluster-scoped
arrivals, the counter protocol and its gmem_counter domain, register groups, the register audit of
the linked image, and one negative case per new clause path (in the style of the reference's
pipec/tests/pipec2/fixtures/negative: one mutation, one clause)."""
import copy
import json

import pytest

from pipelink_b200.pipec2 import contracts, schema
from pipelink_b200.pipec2.model import PipeLinkError
from pipelink_b200.pipec2.profile import PROFILES
from pipelink_b200.pipec2.solve import solve
from pipelink_b200.stages.moe import build as mb

PROFILE = PROFILES["sm_100a"]


def _stages(comp="gate_up_dispatch"):
    return [copy.deepcopy(mb.MANIFESTS[m]) for m in mb.COMPOSITIONS[comp]]


def _solve_inputs(ms, comp="gate_up_dispatch"):
    spec = mb.pipeline_spec(comp, mb.COMPOSITIONS[comp], [])["pipeline"]
    claims, reg_claims, role_warps = {}, {}, {}
    for m in ms:
        for cl in m["claims"]:
            if cl["domain"] == "regs":
                rec = reg_claims.setdefault(cl["handle"], dict(cl, roles=[]))
                rec["roles"] = sorted(set(rec["roles"]) | set(cl["roles"]))
            else:
                claims[cl["handle"]] = {k: v for k, v in cl.items() if k != "roles"}
                if cl["domain"] == "warp":
                    role_warps[cl["roles"][0]] = (cl["handle"], cl["extent"]["const"])
    return claims, spec, list(reg_claims.values()), role_warps


def _solve(ms, comp="gate_up_dispatch", **over):
    claims, spec, reg_claims, role_warps = _solve_inputs(ms, comp)
    kw = dict(depth_priority=spec["depth_priority"], regs_priority=spec["regs_priority"], reg_claims=reg_claims,
              role_warps=role_warps, pipeline_domains=spec["domains"])
    kw.update(over)
    return solve(claims, spec["handles"], PROFILE, **kw)


def test_manifests_validate_and_topology_is_a_cta_pair():
    for m in mb.MANIFESTS.values():
        schema.validate_manifest(copy.deepcopy(m))
    for comp in mb.COMPOSITIONS:
        assert contracts.check_topology(_stages(comp), PROFILE) == (2, (2, 1, 1))


def test_protocol_expansion_counts_arrivals_per_cluster_and_records_the_counter():
    ms = _stages()
    ch = contracts.pair_channels(ms)
    contracts.check_compatibility(ch)
    exp = {e["channel"]: e for e in contracts.expand_protocols(ch, ms, cluster_size=2)}
    assert exp["operands"]["full"]["count"] == 2 and exp["operands"]["full"]["tx_bytes"] == 2 * mb.SLOT_TX
    assert exp["accumulator"]["empty"]["count"] == 16          # eight epilogue warps in each CTA of the pair
    spec = mb.pipeline_spec("gate_up_dispatch", mb.COMPOSITIONS["gate_up_dispatch"], [])["pipeline"]
    (counter,) = contracts.expand_counters(contracts.counter_channels(ms), spec["handles"])
    assert counter["counter"] == ["pipelink_moe_rows_ready", "red.release.gpu", ["ld.acquire.gpu"]]
    assert counter["producers"] == ["moe.comm.dispatch"] and counter["consumers"] == ["moe.load"]
    # without the cluster, two arrivals cannot come from a one-warp role
    with pytest.raises(PipeLinkError, match="L-PROTO"):
        contracts.expand_protocols(ch, ms, cluster_size=1)


def test_solver_places_ring_counters_and_register_groups():
    b, intervals, info = _solve(_stages())
    assert b["pipelink_moe_depth"][0] == 6                      # seven 35,840-byte slots + staging exceed 232,448 bytes
    assert b["pipelink_moe_operands"][0] % 1024 == 0
    assert b["pipelink_moe_warp_epilogue"][0] == 4              # two whole warpgroups behind the helpers' one
    groups = {g["name"]: g for g in info["reg_groups"]}
    assert (groups["helpers"]["warp_lo"], groups["helpers"]["warp_hi"], groups["helpers"]["regs"]) == (0, 4, 56)
    assert (groups["epilogue"]["warp_lo"], groups["epilogue"]["warp_hi"], groups["epilogue"]["regs"]) == (4, 12, 224)
    assert info["launch_regs"] == 168                           # 128 x 56 + 256 x 224 = 384 x 168: the whole pool
    slots = sorted((iv["lo"], iv["hi"]) for iv in intervals["gmem_counter"])
    assert slots[0][1] <= slots[1][0] and slots[-1][1] <= mb.MAX_ROW_TILES + 64
    tm = sorted((iv["lo"], iv["hi"]) for iv in intervals["tmem"])
    assert tm[-1][1] <= 512 and all(a[1] <= c[0] for a, c in zip(tm, tm[1:]))
    # the gate/up composition without dispatch claims no staging: the same depth in less shared memory
    _, _, plain = _solve(_stages("gate_up"), "gate_up")
    assert plain["high_water"]["smem"] < info["high_water"]["smem"]


NEGATIVE = [
    ("mixed cta_group", lambda ms: ms[1]["topology"]["cta_group"].__setitem__("fixed", 1), "L-TOPO", "stages.topology.cta_group"),
    ("cluster shapes differ", lambda ms: ms[3]["topology"]["cluster"].__setitem__("compiled", [4, 1, 1]), "L-TOPO", "stages.topology.cluster"),
    ("counter consumer without producer", lambda ms: ms[2]["endpoints"].pop(0), "L-PAIR", "channels.rows_ready"),
    ("counter release disagrees", lambda ms: ms[2]["endpoints"][0]["protocol"]["counter"].__setitem__("release", "red.release.sys"),
     "L-PROTO", "channels.rows_ready.protocol"),
    ("counter outside gmem", lambda ms: ms[0]["endpoints"][1].__setitem__("space", "smem"), "L-PROTO", "channels.rows_ready.protocol"),
    ("acquire outside the scope's vocabulary", lambda ms: ms[0]["endpoints"][1]["protocol"]["counter"].__setitem__("acquire", "ld.acquire.sys"),
     "L-PROTO", "channels.rows_ready.protocol.acquire"),
    ("payload larger than the slot", lambda ms: [m["endpoints"][0]["ring"].__setitem__("payload_bytes", mb.SLOT + 1024) for m in ms[:2]],
     "L-PROTO", "channels.operands"),
]


@pytest.mark.parametrize("name,mutate,clause,path", NEGATIVE, ids=[n[0] for n in NEGATIVE])
def test_negative_contracts(name, mutate, clause, path):
    ms = _stages()
    mutate(ms)
    spec = mb.pipeline_spec("gate_up_dispatch", mb.COMPOSITIONS["gate_up_dispatch"], [])["pipeline"]
    with pytest.raises(PipeLinkError) as e:
        contracts.check_topology(ms, PROFILE)
        ch = contracts.pair_channels(ms)
        contracts.check_compatibility(ch)
        contracts.expand_protocols(ch, ms, cluster_size=2)
        contracts.expand_counters(contracts.counter_channels(ms), spec["handles"])
    assert any(f.clause_id == clause and f.path.startswith(path) for f in e.value.failures), str(e.value)


def test_counter_slot_must_live_in_the_counter_domain():
    ms = _stages()
    spec = mb.pipeline_spec("gate_up_dispatch", mb.COMPOSITIONS["gate_up_dispatch"], [])["pipeline"]
    spec["handles"]["pipelink_moe_rows_ready"]["domain"] = "smem"
    with pytest.raises(PipeLinkError, match="gmem_counter"):
        contracts.expand_counters(contracts.counter_channels(ms), spec["handles"])


def _drop_comm_regs(ms):
    ms[2]["claims"] = [c for c in ms[2]["claims"] if c["domain"] != "regs"]


def _comm_takes_three_warps(ms):
    for c in ms[2]["claims"]:
        if c["domain"] == "warp":
            c["extent"] = {"const": 3, "per": {}}


def _epilogue_wants_232(ms):
    for c in ms[3]["claims"]:
        if c["domain"] == "regs":
            c["values"] = [232]


# the reference's fixtures 10-12 (a group that does not cover its warpgroup, a group across a
# warpgroup boundary, roles that are no run of whole warpgroups) restated on this pipeline, plus
# the pool itself: 128 x 56 + 256 x 232 registers exceed what a 384-thread launch can be given
REG_NEGATIVE = [("a role left out of every group", _drop_comm_regs),
                ("a group that ends inside a warpgroup", _comm_takes_three_warps),
                ("register pool exceeded", _epilogue_wants_232)]


@pytest.mark.parametrize("name,mutate", REG_NEGATIVE, ids=[n[0] for n in REG_NEGATIVE])
def test_negative_register_groups(name, mutate):
    ms = _stages()
    mutate(ms)
    claims, spec, reg_claims, role_warps = _solve_inputs(ms)
    if name == "register pool exceeded":
        spec["handles"]["pipelink_moe_regs_epilogue"]["values"] = [232]
    with pytest.raises(PipeLinkError) as e:
        solve(claims, spec["handles"], PROFILE, depth_priority=spec["depth_priority"], regs_priority=spec["regs_priority"],
              reg_claims=reg_claims, role_warps=role_warps, pipeline_domains=spec["domains"])
    assert any(f.clause_id == "L-REGS" for f in e.value.failures), str(e.value)


def test_counter_domain_capacity_comes_from_the_pipeline():
    ms = _stages()
    with pytest.raises(PipeLinkError) as e:
        _solve(ms, pipeline_domains={"gmem_counter": {"capacity": 100}})     # 4096 tile counters do not fit 100 slots
    # a domain's capacity is tracked the way the reference tracks it: L-OVERLAP at solve.capacity.<domain>
    assert {(f.clause_id, f.path) for f in e.value.failures} == {("L-OVERLAP", "solve.capacity.gmem_counter")}, str(e.value)


@pytest.fixture(scope="module")
def linked(tmp_path_factory):
    out = tmp_path_factory.mktemp("moe")
    return out, mb.build(out, one_tu=False)      # the one-unit control builds are for timing on a GPU


def test_seven_compositions_link_from_one_set_of_packages(linked):
    out, results = linked
    assert set(results) == {"gate_up", "gate_up_dispatch", "down", "fwd", "fwd_dispatch", "fwd_full", "fwd_full_dispatch"}
    for comp, r in results.items():
        assert (r.threads, tuple(r.cluster), r.tmem_columns, r.regs_cap) == (384, (2, 1, 1), 512, 168)
        assert r.observed[0] <= 168 and r.observed[2] == 0          # register audit: fits the solved launch allocation, no spills
        assert (out / comp / "pipeline.cubin").stat().st_size > 10000
        receipt = json.loads((out / comp / "link.json").read_text())
        # the one-launch forward with dispatch holds the operands ring, the row-store staging and the dispatch
        # ring at once: the solve gives the ring one stage less
        assert receipt["bindings"]["pipelink_moe_depth"] == [5 if comp in ("fwd_dispatch", "fwd_full_dispatch") else 6, "solved"]
        text = (out / comp / "generated" / "dispatch.cu").read_text()
        assert "__cluster_dims__(2, 1, 1)" in text and "tcgen05.alloc.cta_group::2" in text
        assert "setmaxnreg.dec.sync.aligned.u32 56" in text and "setmaxnreg.inc.sync.aligned.u32 224" in text
        assert "barrier.cluster.arrive" in text
    # the dispatch composition carries the counter channel with a real producer
    exp = [e for e in results["gate_up_dispatch"].protocol_expansions if e["kind"] == "counter"]
    assert exp and exp[0]["producers"] == ["moe.comm.dispatch"]
    assert results["gate_up"].dyn_smem_bytes < results["down"].dyn_smem_bytes
    # the one-launch forward: a second counter channel, from the epilogue owner back to the load owner
    exp = {e["channel"]: e for e in results["fwd_dispatch"].protocol_expansions if e["kind"] == "counter"}
    assert exp["hidden_ready"]["producers"] == ["moe.fwd.epilogue"] and exp["rows_ready"]["producers"] == ["moe.comm.dispatch"]
    b = results["fwd_dispatch"].bindings
    slots = sorted((b[h][0], h) for h in ("pipelink_moe_hidden_ready", "pipelink_moe_rows_ready", "pipelink_moe_ticket"))
    assert [s for s, _ in slots] == [0, 4096, 8192]                 # disjoint intervals of the counter workspace
    # the whole forward in one launch: the tail's done-count slot and its named barrier are link-time facts too
    full = results["fwd_full_dispatch"].bindings
    assert full["pipelink_moe_tail_barrier"][0] >= 1 and full["pipelink_moe_ctas_done"][0] == 0
    assert sorted(full[h][0] for h in ("pipelink_moe_hidden_ready", "pipelink_moe_rows_ready", "pipelink_moe_ticket")) == [1, 4097, 8193]
