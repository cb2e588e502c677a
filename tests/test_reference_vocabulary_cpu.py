"""Two stage sources written in the reference's annotation spelling (tests/golden/sources/) packed with THIS
header: the declared sections of the manifests must equal what the reference's own annotation pass emitted
for the same two files (recorded by tests/golden/make_reference_vocabulary.py; the annotation vocabulary is
docs/reference/annotations.md and pipec/include/pipelink/stage.hpp of the reference)."""
import json
from pathlib import Path

import pytest

from pipelink_b200.pipec2 import pack, schema

GOLDEN = Path(__file__).resolve().parent / "golden"
DECLARED = ("stage", "endpoints", "claims", "topology", "hints")


@pytest.mark.parametrize("unit", ["vocabulary", "vocabulary_b"])
def test_header_emits_the_reference_manifest(unit):
    want = json.loads((GOLDEN / f"reference_{unit}_unit.json").read_text())
    got = pack.emit_manifest(GOLDEN / "sources" / f"{unit}.cu")
    for section in DECLARED:
        assert got.get(section) == want.get(section), section
    for key in ("type", "bytes", "align"):
        assert got["params"][key] == want["params"][key]
    # and what this header emitted is a manifest this repository's schema accepts
    got["pipelink_abi"] = want["pipelink_abi"]
    got["payload"] = {"file": "stage.o"}
    schema.validate_manifest(got, where=unit)


def test_vocabulary_units_cover_the_forms():
    """The pin is only as wide as the sources: every protocol kind and claim form is present in them."""
    units = [json.loads((GOLDEN / f"reference_{u}_unit.json").read_text()) for u in ("vocabulary", "vocabulary_b")]
    kinds = {(e.get("protocol") or {}).get("kind") for m in units for e in m["endpoints"]}
    assert {"mbarrier", "call", "counter"} <= kinds      # named barriers: the profile-consumer units of test_reference_sources_cpu
    domains = {c["domain"] for m in units for c in m["claims"]}
    assert {"smem", "mbarrier", "warp", "regs", "gmem_counter"} <= domains
    assert any("empty" not in e["protocol"] for m in units for e in m["endpoints"] if (e.get("protocol") or {}).get("kind") == "mbarrier")
