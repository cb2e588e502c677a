"""``pipec2 pack`` on annotated sources: the manifest a unit's ``PL_*`` annotations emit (host
projection compiled with g++; the reference's scheme, docs/reference/annotations.md), the layout
facts it takes from the compiler, and the failures of a malformed unit. No GPU."""
import json
import textwrap

import pytest

from pipelink_b200.pipec2 import container, link as linker, pack, schema
from pipelink_b200.pipec2.model import PipeLinkError
from pipelink_b200.stages.moe import build as mb

UNIT = """
#include <pipelink/stage.hpp>
struct alignas(16) DemoParams { const float* in; float* out; int count; int pad; };
extern "C" __device__ void org_demo_scale_role(const void* params, unsigned variant);
extern "C" __device__ int pipelink_demo_ring();
PL_STAGE("org.demo-scale", "1.2.0");
PL_PARAMS(DemoParams, in, out, count);
PL_ROLE(scale, org_demo_scale_role, 4);
PL_CLAIM_WARPS(pipelink_demo_warps, scale, 4, 4);
PL_CLAIM(smem, pipelink_demo_ring, pl::per("pipelink_demo_depth", 4096) + pl::units(64), 128);
PL_HINT("note", "unchecked");
%s
#ifndef PIPELINK_EMIT
extern "C" __device__ void org_demo_scale_role(const void* raw, unsigned) {
  const DemoParams& p = *static_cast<const DemoParams*>(raw);
  for (int i = threadIdx.x; i < p.count; i += blockDim.x) p.out[i] = 2.0f * p.in[i] + pipelink_demo_ring();
}
#endif
"""


def _unit(tmp_path, extra=""):
    src = tmp_path / "scale.cu"
    src.write_text(UNIT % extra)
    return src


def test_annotations_emit_a_valid_manifest_with_the_compilers_layout(tmp_path):
    m = pack.emit_manifest(_unit(tmp_path))
    assert m["stage"]["id"] == "org.demo-scale" and m["stage"]["symbol_prefix"] == "org_demo_scale_"
    assert m["stage"]["roles"] == {"scale": {"entry": "org_demo_scale_role", "warps": 4}}
    assert m["params"]["bytes"] == 32 and m["params"]["align"] == 16
    assert [(x["name"], x["offset"], x["bytes"]) for x in m["params"]["members"]] == [("in", 0, 8), ("out", 8, 8), ("count", 16, 4)]
    ring = next(c for c in m["claims"] if c["handle"] == "pipelink_demo_ring")
    assert ring["extent"] == {"const": 64, "per": {"pipelink_demo_depth": 4096}} and ring["align"] == 128
    assert m["hints"] == {"note": "unchecked"} and m["stage"]["variants"] == [{"index": 0, "key": {}}]
    m["pipelink_abi"] = json.loads(json.dumps(mb.ABI))
    schema.validate_manifest(m)
    # a member added to the struct changes the probe
    other = tmp_path / "other.cu"
    other.write_text((UNIT % "").replace("PL_PARAMS(DemoParams, in, out, count)", "PL_PARAMS(DemoParams, in, out, count, pad)"))
    assert pack.emit_manifest(other)["params"]["sha256_of_layout_probe"] != m["params"]["sha256_of_layout_probe"]


def test_pack_reads_the_undefined_symbols_from_the_units_ptx(tmp_path):
    out = pack.pack_cu(_unit(tmp_path), None, tmp_path / "scale.plink")
    m, payload = container.read(out)
    assert m["symbols"]["mechanism"] == "ptx-extern" and m["symbols"]["undefined"] == {"pipelink_demo_ring": "function"}
    assert m["symbols"]["defined_strong"] == ["org_demo_scale_role"]
    assert m["provenance"]["mechanism"] == "annotations" and len(payload) > 0


@pytest.mark.parametrize("extra, clause", [
    ('PL_STAGE("org.second", "1.0.0");', "P-ANNOTATION"),                 # two stages in one unit
    ("PL_NO_PARAMS();", "P-ANNOTATION"),                                    # two parameter blocks
    ("PL_TOPOLOGY(pl::topology()); PL_TOPOLOGY(pl::topology().persistent());", "P-ANNOTATION"),
    ('extern "C" __device__ int bad_entry(int); PL_ROLE(bad, bad_entry, 1);', "P-COMPILE"),   # not the entry signature
])
def test_malformed_units_fail_with_a_clause(tmp_path, extra, clause):
    with pytest.raises(PipeLinkError) as err:
        pack.emit_manifest(_unit(tmp_path, extra))
    assert err.value.failures[0].clause_id == clause


TENSOR_EXPORT = '''PL_EXPORT_TENSOR(tile, pl::identity{"tile", "work", "done", "f32", "plain", {{"m", 0, 16}, {"n", 0, 8}}},
    pl::placement{"smem", "byte", {"address"}, [](int m, int n) { return std::array<int, 1>{%s}; },
                  pl::coord{"m", 0, 16}, pl::coord{"n", 0, 8}},
    pl::strings{"smem_load_scalar"}, pl::readiness{"ready", "done"}, pl::fixed_bindings{},
    pl::lends{pl::smem("store", 512, 16, "pipelink_demo_store", "scale", "work", "done")}, pl::calls{"produce", "release"});'''


@pytest.mark.parametrize("body, address", [
    ("4 * (8 * m + n) + 64", ["add", ["add", ["mulc", 32, ["coord", "m"]], ["mulc", 4, ["coord", "n"]]], ["const", 64]]),      # affine
    ("4 * ((8 * m + n) ^ (m >> 1))", None),                                                                                   # XOR swizzle
    ("4 * (8 * (m / 2) + 4 * (m % 2) + n / 2) + 256 * (n % 2)", None),                                                         # bit permutation
])
def test_a_placement_lambda_is_solved_to_an_expression(tmp_path, body, address):
    """Whatever family the map falls in, the printed expression reproduces the lambda on its whole domain."""
    from pipelink_b200.pipec2 import tensor
    m = pack.emit_manifest(_unit(tmp_path, TENSOR_EXPORT % body))
    expr = m["tensor"]["exports"][0]["placements"][0]["components"]["address"]
    if address is not None:
        assert expr == address
    else:
        assert expr[0] in ("toint", "add", "mulc", "modc", "divc")
    for mm in range(16):
        for nn in range(8):
            want = eval(body.replace("/", "//"), {"m": mm, "n": nn})
            assert tensor.evaluate(expr, {"m": mm, "n": nn}) == want, (mm, nn)


def test_a_map_of_neither_family_is_refused(tmp_path):
    with pytest.raises(PipeLinkError) as err:
        pack.emit_manifest(_unit(tmp_path, TENSOR_EXPORT % "m * n"))
    assert err.value.failures[0].clause_id == "P-ANNOTATION" and "neither integer-affine nor XOR-linear" in str(err.value)


def test_moe_units_state_the_sizes_their_structs_have():
    ms = mb.manifests()
    sizes = {name: (m["params"]["bytes"], m["params"]["align"]) for name, m in ms.items()}
    assert sizes == {"load": (576, 64), "mma": (48, 16), "comm_none": (0, 1), "comm_dispatch": (112, 16),
                     "epilogue_swiglu": (80, 16), "epilogue_rows": (96, 16), "fwd_load": (1152, 64),
                     "fwd_mma": (96, 16), "fwd_epilogue": (176, 16), "fwd_epilogue_combine": (256, 16)}
    # the members an owner reads cover its block up to tail padding
    for m in ms.values():
        if m["params"]["bytes"]:
            last = max(m["params"]["members"], key=lambda x: x["offset"])
            assert m["params"]["bytes"] - (last["offset"] + last["bytes"]) < m["params"]["align"]


def test_a_symbol_no_handle_binds_fails_the_link(tmp_path):
    """L-SYM: a stage that calls a pipelink_* function the pipeline does not bind."""
    import copy
    ms = {k: copy.deepcopy(v) for k, v in mb.manifests().items()}
    for name, m in ms.items():
        m["symbols"].update(mechanism="ptx-extern", defined_weak=[], undefined={})
        m["payload"] = {"file": "stage.o"}
    ms["load"]["symbols"]["undefined"] = {"pipelink_moe_depth": "function", "pipelink_moe_missing": "function"}
    members = mb.COMPOSITIONS["gate_up"]
    for name in members:
        (tmp_path / f"{name}.plink").write_bytes(container.pack(ms[name], b"x"))
    stages = [{"stage_id": ms[n]["stage"]["id"], "artifact_path": f"{n}.plink"} for n in members]
    spec = tmp_path / "p.json"
    spec.write_text(json.dumps(mb.pipeline_spec("gate_up", members, stages)))
    with pytest.raises(PipeLinkError) as err:
        linker.link(spec, tmp_path / "out", device_link=False)
    assert [(f.clause_id, f.path) for f in err.value.failures] == [("L-SYM", "moe.load.symbols.pipelink_moe_missing")]
    ms["load"]["symbols"]["undefined"] = {"pipelink_moe_depth": "function"}
    ms["mma"]["symbols"]["defined_strong"].append("moe_load_role")
    for name in members:
        (tmp_path / f"{name}.plink").write_bytes(container.pack(ms[name], b"x"))
    with pytest.raises(PipeLinkError) as err:
        linker.link(spec, tmp_path / "out", device_link=False)
    assert err.value.failures[0].clause_id == "L-SYM" and "two stages" in err.value.failures[0].message
