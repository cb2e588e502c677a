"""The reference's `examples/ring-pipeline` through this link driver: the two manifests were emitted
by the REFERENCE's annotation pass from its own sources, the pipeline descriptions are the ones its
build.py writes (tests/golden/make_reference_examples.py recorded both, and what the reference's
front end solves). This driver must accept the documents as they are and solve them to the same
ring depth, launch shape, warp map, protocol expansion and per-domain high-water marks."""
import copy
import json
from pathlib import Path

import pytest

from pipelink_b200.pipec2 import link as linker, schema

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_ring_pipeline.json").read_text())


@pytest.mark.parametrize("name", sorted(GOLDEN["pipelines"]))
def test_ring_pipeline_solves_as_the_reference_solves_it(name):
    manifests = copy.deepcopy(GOLDEN["manifests"])
    doc = copy.deepcopy(GOLDEN["pipelines"][name])
    for m in manifests:
        schema.validate_manifest(m)
    schema.validate_pipeline(doc)
    fe = linker.front_end(manifests, doc["pipeline"])
    want = GOLDEN["reference"][name]
    assert {h: fe["bindings"][h][0] for h in want["depths"]} == want["depths"]
    warp_map = {role: [fe["bindings"][h][0] + off, fe["bindings"][h][0] + off + warps] for role, (h, warps, off) in fe["role_warps"].items()}
    assert warp_map == want["warp_map"]
    assert 32 * sum(w for _, w, _ in fe["role_warps"].values()) == want["threads"]
    assert fe["solver"]["high_water"]["smem"] == want["high_water"]["smem"] == want["dyn_smem_bytes"]
    assert list(fe["cluster"]) == want["cluster"]
    extents = {iv["handle"]: iv["hi"] - iv["lo"] for ivs in fe["intervals"].values() for iv in ivs}
    # the reference counts barrier claims in bytes (16 per slot), this driver in slots
    for handle, size in want["extents"].items():
        scale = 16 if handle in ("pipelink_ring_full", "pipelink_ring_empty") else 1
        assert extents[handle] * scale == size, handle
    exp = next(e for e in fe["expansions"] if e["channel"] == "tile_ring")
    assert (exp["full"]["count"], exp["empty"]["count"], exp["full"]["tx_bytes"]) == (
        want["arrive_full"], want["arrive_empty"], want["tx_bytes"])
