"""The link driver without a GPU: container, contracts, solver, code generation, LTO link."""
import copy
import json
from pathlib import Path

import pytest

from pipelink_b200.pipec2 import canonjson, container, contracts, link as linker, schema
from pipelink_b200.pipec2.model import CLAUSES, PipeLinkError
from pipelink_b200.pipec2.profile import PROFILES
from pipelink_b200.pipec2.solve import solve
from pipelink_b200.stages.gemm3 import build as g3


def test_canonical_json_and_container_round_trip(tmp_path):
    assert canonjson.dumps({"b": 1, "a": [1, 2]}) == '{"a":[1,2],"b":1}\n'
    m = copy.deepcopy(g3.MANIFESTS["load"])
    data = container.pack(m, b"payload-bytes")
    assert data == container.pack(copy.deepcopy(g3.MANIFESTS["load"]), b"payload-bytes")   # reproducible
    back, payload = container.read(data)
    assert payload == b"payload-bytes" and back["stage"]["id"] == "gemm.load" and len(back["payload"]["sha256"]) == 64
    with pytest.raises(PipeLinkError, match="P-CONTAINER"):
        container.pack(back, b"x")        # a packed manifest already carries a digest
    with pytest.raises(PipeLinkError, match="P-CONTAINER"):
        container.read(data[:-20])


def test_manifests_validate_and_symbol_prefix_rule():
    for m in g3.MANIFESTS.values():
        schema.validate_manifest(copy.deepcopy(m))
    assert schema.symbol_prefix("gemm.epilogue.bias-silu") == "gemm_epilogue_bias_silu_"
    bad = copy.deepcopy(g3.MANIFESTS["mma"])
    bad["stage"]["symbol_prefix"] = "other_"           # the prefix is derived from the stage id
    with pytest.raises(PipeLinkError, match="P-SYM"):
        schema.validate_manifest(bad)
    bad = copy.deepcopy(g3.MANIFESTS["mma"])
    bad["stage"]["entry_abi"] = "v1"
    with pytest.raises(PipeLinkError, match="L-ENTRYABI"):
        schema.validate_manifest(bad)


def _channels(ms):
    ch = contracts.pair_channels(ms)
    contracts.check_compatibility(ch)
    return ch


def _ep(m, name):
    return next(e for e in m["endpoints"] if e["name"] == name)


# negative corpus in the style of pipec/tests/pipec2/fixtures/negative: one mutation, one clause
# (ms[0] = load, ms[1] = mma; both hold an end of `operands`)
NEGATIVE = [
    ("missing consumer", lambda ms: ms[1]["endpoints"].remove(_ep(ms[1], "operands")), "L-PAIR", "channels.operands"),
    ("scope differs", lambda ms: _ep(ms[1], "operands").__setitem__("scope", "cluster"), "L-PAIR", "channels.operands.endpoint.scope"),
    ("layout differs", lambda ms: _ep(ms[1], "operands")["layout"]["stride"].__setitem__(1, [256]), "L8", "channels.operands.layout"),
    ("swizzle differs", lambda ms: _ep(ms[1], "operands")["layout"].__setitem__("swizzle", {"B": 2, "M": 4, "S": 3}), "L8", "channels.operands.layout"),
    ("tx bytes differ", lambda ms: _ep(ms[1], "operands")["protocol"]["full"].__setitem__("tx_bytes", 1024), "L-PROTO", "channels.operands.protocol"),
    ("arrive count impossible", lambda ms: [_ep(m, "operands")["protocol"]["empty"]["arrive"].__setitem__("count", 7) for m in ms[:2]],
     "L-PROTO", "channels.operands.protocol.empty.arrive.count"),
    ("two materializers", lambda ms: _ep(ms[0], "operands")["protocol"]["init"].__setitem__("materializer", "load"),
     "L-PROTO", "channels.operands.protocol.init"),
]


@pytest.mark.parametrize("name,mutate,clause,path", NEGATIVE, ids=[n[0] for n in NEGATIVE])
def test_negative_contracts(name, mutate, clause, path):
    ms = [copy.deepcopy(g3.MANIFESTS[k]) for k in ("load", "mma", "epilogue_bias_silu")]
    mutate(ms)
    with pytest.raises(PipeLinkError) as e:
        ch = _channels(ms)
        contracts.expand_protocols(ch, ms)
    assert any(f.clause_id == clause and f.path.startswith(path) for f in e.value.failures), str(e.value)


def test_layout_identity_ignores_mode_nesting():
    a = {"elem_bits": 8, "shape": [[2], [128], [128]], "stride": [[16384], [128], [1]], "swizzle": None}
    b = {"elem_bits": 8, "shape": [[2, 128, 128]], "stride": [[16384, 128, 1]], "swizzle": None}
    c = {"elem_bits": 8, "shape": [[32768]], "stride": [[1]], "swizzle": None}
    assert contracts.canonical_layout(a) == contracts.canonical_layout(b) == contracts.canonical_layout(c)


def _claims_and_handles(values=(6, 5, 4, 3, 2)):
    spec = g3.pipeline_spec([], values=values)["pipeline"]
    claims = {}
    for m in g3.MANIFESTS.values():
        for cl in m["claims"]:
            claims[cl["handle"]] = {k: v for k, v in cl.items() if k != "roles"}
    return claims, spec["handles"]


def test_solver_picks_largest_depth_that_fits_and_packs_without_overlap():
    claims, handles = _claims_and_handles(values=(8, 7, 6, 5, 4, 3, 2))
    bindings, intervals, info = solve(claims, handles, PROFILES["sm_100a"], depth_priority=["pipelink_gemm_depth"])
    depth = bindings["pipelink_gemm_depth"][0]
    assert depth == 6                       # 7 x 33,792 B does not fit 232,448 B of shared memory
    smem = [(iv["lo"], iv["hi"]) for iv in intervals["smem"]] + [(16 * iv["lo"], 16 * iv["hi"]) for iv in intervals["mbarrier"]]
    smem.sort()
    assert all(a[1] <= b[0] for a, b in zip(smem, smem[1:])) and smem[-1][1] <= 232448
    assert bindings["pipelink_gemm_operands"][0] % 1024 == 0
    tm = sorted((iv["lo"], iv["hi"]) for iv in intervals["tmem"])
    assert tm[0][0] % 32 == 0 and tm[0][1] <= tm[1][0] and tm[1][1] <= 512
    warps = sorted((iv["lo"], iv["hi"]) for iv in intervals["warp"])
    assert warps[0][0] == 0 and all(a[1] == b[0] for a, b in zip(warps, warps[1:])) and warps[-1][1] == 6
    assert bindings["pipelink_gemm_warp_epilogue"][0] % 4 == 0
    assert info["high_water"]["smem"] <= 232448


def test_solver_forced_binding_and_unsat_diagnostics():
    claims, handles = _claims_and_handles()
    b, _, _ = solve(claims, handles, PROFILES["sm_100a"], forced={"pipelink_gemm_depth": 2})
    assert b["pipelink_gemm_depth"] == [2, "forced"]
    with pytest.raises(PipeLinkError, match="L-HANDLE"):
        solve(claims, handles, PROFILES["sm_100a"], forced={"pipelink_gemm_depth": 9})
    claims, handles = _claims_and_handles(values=(8,))      # only candidate does not fit
    with pytest.raises(PipeLinkError) as e:
        solve(claims, handles, PROFILES["sm_100a"])
    assert {f.clause_id for f in e.value.failures} <= set(CLAUSES)


@pytest.fixture(scope="module")
def linked(tmp_path_factory):
    out = tmp_path_factory.mktemp("gemm3")
    return out, g3.build(out)


def test_link_three_stage_gemm(linked):
    out, r = linked
    assert r.kernel_symbol == "pipelink_kernel" and r.threads == 192 and r.tmem_columns == 256
    assert r.bindings["pipelink_gemm_depth"] == [6, "solved"]
    assert r.dyn_smem_bytes <= 232448 and r.dyn_smem_bytes >= 6 * g3.SLOT
    # stages in the order of their ids, each block on the target's 64-byte parameter alignment (the reference's rule)
    assert [e[:3] for e in r.params["entries"]] == [["gemm.epilogue.bias-silu", 0, 32], ["gemm.load", 64, 320], ["gemm.mma", 384, 16]]
    assert r.params["total_bytes"] == 448
    kinds = {(e["channel"], e["kind"]) for e in r.protocol_expansions}
    assert kinds == {("operands", "mbarrier"), ("accumulator", "mbarrier")}
    link_dir = out / "link"
    receipt = json.loads((link_dir / "link.json").read_text())
    assert receipt["bindings"]["pipelink_gemm_depth"][0] == 6 and set(receipt["generated_hashes"]) == {"binding_stub.cu", "dispatch.cu"}
    stub = (link_dir / "generated" / "binding_stub.cu").read_text()
    assert 'extern "C" __device__ int pipelink_gemm_depth() { return 6; }' in stub
    dispatch = (link_dir / "generated" / "dispatch.cu").read_text()
    assert "pipelink_kernel" in dispatch and "gemm_mma_role" in dispatch and "tcgen05.alloc" in dispatch
    assert (link_dir / "pipeline.cubin").stat().st_size > 10000 and (link_dir / "one_tu.cubin").stat().st_size > 10000


def test_link_rejects_undeclared_handle_and_relinks_with_forced_depth(linked, tmp_path):
    out, _ = linked
    spec = json.loads((out / "pipeline.json").read_text())
    for s in spec["pipeline"]["stages"]:
        s["artifact_path"] = str(out / s["artifact_path"])
    bad = copy.deepcopy(spec)
    del bad["pipeline"]["handles"]["pipelink_gemm_sf"]
    (tmp_path / "bad.json").write_text(json.dumps(bad))
    with pytest.raises(PipeLinkError, match="L-HANDLE"):
        linker.link(tmp_path / "bad.json", tmp_path / "bad", device_link=False)
    spec["pipeline"]["forced_bindings"] = {"pipelink_gemm_depth": 3}
    (tmp_path / "d3.json").write_text(json.dumps(spec))
    r = linker.link(tmp_path / "d3.json", tmp_path / "d3", device_link=False)
    assert r.bindings["pipelink_gemm_depth"] == [3, "forced"] and r.dyn_smem_bytes < 4 * g3.SLOT


def test_cli_verbs(linked, capsys):
    from pipelink_b200.pipec2 import cli
    out, _ = linked
    assert cli.main(["clauses"]) == 0
    assert "L-PROTO" in capsys.readouterr().out
    assert cli.main(["inspect", str(out / "mma.plink")]) == 0
    assert "gemm.mma" in capsys.readouterr().out
    # the flags the reference's example scripts pass (examples/contract-gallery/check.py:57-90)
    assert cli.main(["clauses", "--json"]) == 0
    assert set(json.loads(capsys.readouterr().out)) >= {"L-PROTO", "L-TOPO", "L-HANDLE", "L-PARAMS", "L-PHASE"}
    assert cli.main(["inspect", str(out / "mma.plink"), "--json"]) == 0
    assert json.loads(capsys.readouterr().out)["stage"]["id"] == "gemm.mma"
    assert cli.main(["link", str(out / "pipeline.json"), "--out-dir", str(out / "cli_link"), "--no-device-link"]) == 0
    assert json.loads(capsys.readouterr().out)["threads"] == 192
    broken = json.loads((out / "pipeline.json").read_text())
    broken["pipeline"]["topology"]["persistent"] = not broken["pipeline"]["topology"].get("persistent", False)
    (out / "broken.json").write_text(json.dumps(broken))
    assert cli.main(["link", str(out / "broken.json"), "--out-dir", str(out / "cli_broken"), "--no-device-link"]) == 1
    import re
    # the structured prefix their checker reads clause tokens from, never the prose
    assert re.findall(r"(?:^pipec2: |; )\[([A-Z][A-Z0-9]*(?:-[A-Z0-9]+)*)\] ", capsys.readouterr().err, re.M) == ["L-TOPO"] * 3


def test_config0_oracle_is_finite_and_shaped():
    from oracle import gemm3
    case = gemm3.make_case(256, 256, 256)
    ref = gemm3.expected(case)
    assert ref.shape == (256, 256) and gemm3.compare(ref, ref)["violations"] == 0


# ---- held to the reference's own linker front end -------------------------------------------
# tests/golden/gemm3_reference_linker.json records what pipec2 of the reference tree answers for
# THIS repo's packages and pipeline variants (tests/golden/make_linker_golden.py made it).
GOLDEN = json.loads((Path(__file__).parent / "golden" / "gemm3_reference_linker.json").read_text())


@pytest.mark.parametrize("case", sorted(GOLDEN["solutions"]))
def test_solution_tiers_equal_the_reference_linker(linked, tmp_path, case):
    from tests.golden import linker_cases
    out, _ = linked
    stages = json.loads((out / "pipeline.json").read_text())["pipeline"]["stages"]
    for s in stages:
        s["artifact_path"] = str(out / s["artifact_path"])
    spec = tmp_path / "pipeline.json"
    spec.write_text(json.dumps(g3.pipeline_spec(stages, **linker_cases.SOLVE_CASES[case])))
    r = linker.link(spec, tmp_path / "link", device_link=False)
    want = GOLDEN["solutions"][case]
    assert {h: r.bindings[h][0] for h in want["depths"]} == want["depths"]
    assert r.threads == want["threads"] and list(r.cluster) == want["cluster"]
    hw = {d: max(iv["hi"] for iv in ivs) for d, ivs in r.intervals.items()}
    assert hw["tmem"] == want["high_water"]["tmem"] and hw["warp"] == want["high_water"]["warp"]
    # this linker adds one 16-byte slot through which dispatch publishes the TMEM base; without it
    # the shared-memory high-water mark is the reference's
    slot = r.bindings[linker.TMEM_SLOT_HANDLE][0]
    others = max(iv["hi"] * (16 if d == "mbarrier" else 1) for d in ("smem", "mbarrier") for iv in r.intervals[d]
                 if iv["handle"] != linker.TMEM_SLOT_HANDLE)
    assert others == want["dyn_smem_bytes"] and r.dyn_smem_bytes == max(others, slot + 16) <= want["dyn_smem_bytes"] + 16
    roles = {x["role"]: [x["warp_lo"], x["warp_hi"]] for x in r.roles}
    assert roles == want["warp_map"]
    ext = {iv["handle"]: (iv["hi"] - iv["lo"]) * (16 if d == "mbarrier" else 1) for d, ivs in r.intervals.items() for iv in ivs}
    for handle, n in want["extents"].items():
        assert ext[handle] == n, handle


@pytest.mark.parametrize("case", sorted(GOLDEN["negative"]))
def test_negative_clause_ids_equal_the_reference_linker(case):
    from tests.golden import linker_cases
    ms = linker_cases.mutated(g3.MANIFESTS, case)
    with pytest.raises(PipeLinkError) as e:
        ch = _channels(ms)
        contracts.expand_protocols(ch, ms)
    assert sorted({f.clause_id for f in e.value.failures}) == GOLDEN["negative"][case], str(e.value)
