"""The reference's 19 negative link fixtures (pipec/tests/pipec2/fixtures/negative/*.json), run
through this link driver. Each fixture is one mutation of a valid base document; the mutated
document must be rejected with the fixture's clause id at a path that contains the fixture's
expected path, at the phase the fixture names (schema / protocol expansion / symbol check / solve),
and the un-mutated bases must pass every phase. The documents and the reference's own answers were
recorded from the reference (tests/golden/make_reference_negatives.py)."""
import copy
import json
from pathlib import Path

import pytest

from pipelink_b200.pipec2 import contracts, link as linker, schema
from pipelink_b200.pipec2.model import PipeLinkError

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_negative_fixtures.json").read_text())
CASES = {c["file"]: c for c in GOLDEN["cases"]}


def _mutated(case):
    raw = copy.deepcopy(GOLDEN["bases"][case["base"]])
    for path in case["paths"]:
        target = raw
        for part in path[:-1]:
            target = target[part]
        target[path[-1]] = copy.deepcopy(case["value"])
    return raw


def _symbol_manifests(raw):
    """The symbol fixtures are bare symbol tables: one manifest per table, nothing else in it."""
    out = []
    for stage_id, table in raw["tables"].items():
        out.append({"stage": {"id": stage_id, "symbol_prefix": raw["prefixes"][stage_id]},
                    "symbols": {"defined_strong": list(table.get("strong", [])), "defined_weak": list(table.get("weak", [])),
                                "undefined": {u: "function" for u in table.get("undefined", [])}}})
    return out


def run_phase(phase, raw, case):
    if phase == "symbols.check":
        return linker._check_symbols(_symbol_manifests(raw), {})
    if phase == "schema.stage":
        return schema.validate_manifest(raw["stages"][case.get("stage_index", 0)])
    if phase == "schema.pipeline":
        return schema.validate_pipeline(raw["pipeline"])
    for m in raw["stages"]:
        schema.validate_manifest(m)
    schema.validate_pipeline(raw["pipeline"])
    if phase == "protocol.expand":
        channels = contracts.pair_channels(raw["stages"])
        contracts.check_compatibility(channels)
        return contracts.expand_protocols(channels, raw["stages"], 1)
    assert phase == "solve"
    return linker.front_end(raw["stages"], raw["pipeline"]["pipeline"])


@pytest.mark.parametrize("base", sorted(GOLDEN["bases"]))
def test_the_reference_bases_pass(base):
    raw = copy.deepcopy(GOLDEN["bases"][base])
    phases = {c["phase"] for c in GOLDEN["cases"] if c["base"] == base}
    for phase in sorted(phases):
        run_phase(phase, raw, {"stage_index": 0})


@pytest.mark.parametrize("name", sorted(CASES))
def test_reference_negative_fixture(name):
    case = CASES[name]
    # the recording itself: the reference answers its own fixture as the fixture expects
    assert {f[0] for f in case["reference_failures"]} == {case["expected_clause"]}
    assert any(case["expected_path"] in f[1] for f in case["reference_failures"])
    with pytest.raises(PipeLinkError) as err:
        run_phase(case["phase"], _mutated(case), case)
    got = [(f.clause_id, f.path) for f in err.value.failures]
    assert {c for c, _ in got} == {case["expected_clause"]}, got
    assert any(case["expected_path"] in p for _, p in got), got


def test_a_materializer_this_build_cannot_generate_is_refused_at_link():
    """Both ends agree on a stage-side barrier initialiser: a valid contract (the reference accepts it)
    that this build's code generator does not implement; the link says so instead of generating
    a dispatch kernel that skips the initialisation."""
    raw = copy.deepcopy(GOLDEN["bases"]["barrier"])
    for st in raw["stages"]:
        st["endpoints"][0]["protocol"]["init"]["materializer"] = "stage"
    run_phase("protocol.expand", raw, {})
    with pytest.raises(PipeLinkError) as err:
        linker.front_end(raw["stages"], raw["pipeline"]["pipeline"])
    assert [(f.clause_id, f.path) for f in err.value.failures] == [("L-OWNER", "channels.ring.protocol.init")]
