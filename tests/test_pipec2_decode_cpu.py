"""The decode interpreter's two owners through the link driver, without a GPU: manifests from the
annotations, the solved shared-memory map, the warp tiling the device code relies on, the
one-way `instructions` hand-off, and a ring that no longer fits."""
import copy
import json

import pytest

from pipelink_b200.pipec2 import contracts, link as linker, schema
from pipelink_b200.pipec2.model import PipeLinkError
from pipelink_b200.stages.decode import build as db


def _stages():
    return [copy.deepcopy(db.manifests()[n]) for n in db.STAGES]


def test_decode_owners_state_their_contract():
    ms = _stages()
    for m in ms:
        schema.validate_manifest(m)
    assert {m["stage"]["id"]: {r: v["warps"] for r, v in m["stage"]["roles"].items()} for m in ms} == {
        "decode.stream": {"stream": 1}, "decode.interpret": {"interpret": 16}}
    sizes = {m["stage"]["id"]: (m["params"]["bytes"], m["params"]["align"]) for m in ms}
    assert sizes == {"decode.stream": (512, 64), "decode.interpret": (256, 16)}       # two tensor maps + the 256-byte argument block
    ch = contracts.pair_channels(ms)
    contracts.check_compatibility(ch)
    exp = {e["channel"]: e for e in contracts.expand_protocols(ch, ms, 1)}
    assert exp["weights"]["full"]["count"] == 1 and exp["weights"]["empty"]["count"] == 16
    assert exp["weights"]["full"]["tx_bytes"] == 32768
    assert exp["instructions"]["empty"] is None and exp["instructions"]["full"]["by"] == "interpret"


def test_decode_image_solves_to_the_library_kernels_map():
    ms = _stages()
    spec = db.pipeline_spec([])["pipeline"]
    fe = linker.front_end(ms, spec)
    b = {k: v[0] for k, v in fe["bindings"].items()}
    assert b["pipelink_dec_depth"] == 6 and b["pipelink_dec_ring"] == 0
    assert (b["pipelink_dec_warp_interpret"], b["pipelink_dec_warp_stream"], b["pipelink_dec_named_barrier"]) == (0, 16, 1)
    assert fe["solver"]["high_water"]["smem"] <= 232448 - 1024          # room for the roles' static shared memory
    # seven stages do not fit beside the partial sums, the attention workspace and the instruction copy
    spec7 = db.pipeline_spec([], values=(7,))["pipeline"]
    with pytest.raises(PipeLinkError) as err:
        linker.front_end(_stages(), spec7)
    assert {f.clause_id for f in err.value.failures} <= {"L-BUDGET", "L-OVERLAP"}


def test_interpreter_warps_must_come_first():
    """The interpreter's code takes threadIdx.x as its thread index: the pipeline pins its warps to 0-15."""
    spec = db.pipeline_spec([])["pipeline"]
    assert spec["forced_bindings"] == {"pipelink_dec_warp_interpret": 0, "pipelink_dec_warp_stream": 16}
    spec["forced_bindings"]["pipelink_dec_warp_stream"] = 3
    with pytest.raises(PipeLinkError):
        linker.front_end(_stages(), spec)


def test_decode_image_links(tmp_path):
    r = db.build(tmp_path, one_tu=False)
    assert (r.threads, r.bindings["pipelink_dec_depth"][0], r.tmem_columns) == (544, 6, 0)
    assert (tmp_path / "link" / "pipeline.cubin").stat().st_size > 10000
    receipt = json.loads((tmp_path / "link" / "link.json").read_text())
    assert [e[0] for e in receipt["params"]["entries"]] == ["decode.interpret", "decode.stream"]      # in the order of the stage ids
    text = (tmp_path / "link" / "generated" / "dispatch.cu").read_text()
    assert "decode_stream_role" in text and "decode_interpret_role" in text
