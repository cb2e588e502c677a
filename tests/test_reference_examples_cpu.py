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


# ---------------------------------------------------------------- examples/contract-gallery
GALLERY = json.loads((Path(__file__).parent / "golden" / "reference_contract_gallery.json").read_text())


def _this_driver(case):
    """The clause(s) this driver raises for a gallery case, or "OK" with the solved launch shape."""
    from pipelink_b200.pipec2.model import PipeLinkError
    manifests = [copy.deepcopy(GALLERY["producer"]), copy.deepcopy(case["manifest"])]
    doc = copy.deepcopy(case["pipeline"])
    try:
        for m in manifests:
            schema.validate_manifest(m)
        schema.validate_pipeline(doc)
        fe = linker.front_end(manifests, doc["pipeline"])
    except PipeLinkError as err:
        return sorted({f.clause_id for f in err.failures}), None
    return "OK", {"threads": 32 * sum(w for _, w, _ in fe["role_warps"].values()), "dyn_smem_bytes": fe["solver"]["high_water"]["smem"]}


@pytest.mark.parametrize("name", sorted(n for n, c in GALLERY["cases"].items() if c["phase"] == "link"))
def test_contract_gallery_cases_end_as_the_reference_ends_them(name):
    """One unchanged producer package against the original consumer, a replacement, and consumers
    with one wrong contract each (the reference's third tutorial): the documents its annotation pass
    emitted must link here where they link there (same launch shape) and fail with the same clause
    where they fail there (recorded by tests/golden/make_reference_contract_gallery.py, which runs
    the reference itself)."""
    case = GALLERY["cases"][name]
    got, launch = _this_driver(case)
    if case["reference"] == "OK":
        assert case["expected_clause"] is None and got == "OK" and launch == case["launch"]
    else:
        want = sorted({f["clause"] for f in case["reference"]})
        assert want == [case["expected_clause"]]          # the reference's own table agrees with what it did here
        assert got == want


def test_contract_gallery_pack_time_case_is_recorded():
    """`init.cu` names a consumer warp as the barrier initialiser although the dispatch kernel
    materialises the ring: the reference refuses it while packing (P-INIT), so there is no
    manifest to link. This driver's annotation pass has no producer/consumer init-warp field to get
    wrong; the case is kept as a record of the reference's behaviour."""
    case = GALLERY["cases"]["init"]
    assert case["phase"] == "pack" and case["manifest"] is None
    assert [f["clause"] for f in case["reference"]] == ["P-INIT"]


# ---------------------------------------------------------------- examples/hello-callable
HELLO = json.loads((Path(__file__).parent / "golden" / "reference_hello_callable.json").read_text())


def test_hello_callable_links_as_the_reference_links_it():
    """The reference's first tutorial: a role-less provider and a caller joined by a call channel.
    Its own annotation pass emitted the manifests (call endpoints spell whole C declarations there);
    this driver pairs the ends, derives the reference's launch shape and parameter total, and plans the
    trampoline between the two declared functions."""
    manifests, doc = copy.deepcopy(HELLO["manifests"]), copy.deepcopy(HELLO["pipeline"])
    for m in manifests:
        schema.validate_manifest(m)
    schema.validate_pipeline(doc)
    fe = linker.front_end(manifests, doc["pipeline"])
    want = HELLO["reference"]
    warp_map = {role: [fe["bindings"][h][0] + off, fe["bindings"][h][0] + off + warps] for role, (h, warps, off) in fe["role_warps"].items()}
    assert warp_map == want["warp_map"]
    assert 32 * sum(w for _, w, _ in fe["role_warps"].values()) == want["threads"] == 128
    assert fe["solver"]["high_water"].get("smem", 0) == want["dyn_smem_bytes"] == 0
    assert fe["params"]["total_bytes"] == want["params"]["total_bytes"]
    mine = {e[0]: (e[2], e[3]) for e in fe["params"]["entries"]}
    assert mine == {e[0]: (e[2], e[3]) for e in want["params"]["entries"]}            # bytes and alignment per stage
    (call,) = [e for e in fe["expansions"] if e["kind"] == "call"]
    assert call["trampoline"] == {"caller": "pipelink_call_scale", "provider": "hello_scale", "signature": "float(float)"}
    from pipelink_b200.pipec2 import codegen
    stub = codegen.binding_stub(fe["bindings"], [call["trampoline"]])
    assert 'extern "C" __device__ float pipelink_call_scale(float a0) { return hello_scale(a0); }' in stub


# ---------------------------------------------------------------- examples/profile-consumer
PROFILE_CONSUMER = json.loads((Path(__file__).parent / "golden" / "reference_profile_consumer.json").read_text())


@pytest.mark.parametrize("name", sorted(PROFILE_CONSUMER["cases"]))
def test_profile_consumer_ends_as_the_reference_ends_it(name):
    """Three stages (a scheduler and two instructions) that hand a shared-memory page over through a
    named barrier and a grid-scoped counter; the pages are claims of a pipeline-defined page domain
    living in mutually exclusive phases, so they may share page 1. The manifests come from the
    reference's annotation pass; tests/golden/make_reference_profile_consumer.py recorded what the
    reference's front end does with the shipped pipeline description and with four one-line changes."""
    from pipelink_b200.pipec2.model import PipeLinkError
    case = PROFILE_CONSUMER["cases"][name]
    manifests, doc, want = copy.deepcopy(PROFILE_CONSUMER["manifests"]), copy.deepcopy(case["pipeline"]), case["reference"]
    try:
        for m in manifests:
            schema.validate_manifest(m)
        schema.validate_pipeline(doc)
        fe = linker.front_end(manifests, doc["pipeline"])
    except PipeLinkError as err:
        assert "failures" in want, f"the reference links this; here: {err}"
        assert sorted({f.clause_id for f in err.failures}) == sorted({f["clause"] for f in want["failures"]})
        return
    assert "failures" not in want
    assert 32 * sum(w for _, w, _ in fe["role_warps"].values()) == want["threads"]
    assert fe["solver"]["high_water"]["smem"] == want["dyn_smem_bytes"]
    warp_map = {role: [fe["bindings"][h][0] + off, fe["bindings"][h][0] + off + warps] for role, (h, warps, off) in fe["role_warps"].items()}
    assert warp_map == want["warp_map"]
    # every claim where the reference puts it, in the reference's units (pages and barrier slots in bytes)
    placed = {}
    for domain, ivs in fe["intervals"].items():
        scale = linker.profile_scale(fe["profile"], doc["pipeline"], domain)
        for iv in ivs:
            placed[iv["handle"]] = [iv["lo"] * scale, iv["hi"] * scale]
    for ivs in want["intervals"].values():
        for handle, lo, hi in ivs:
            assert placed[handle] == [lo, hi], handle
    assert [e["named_barrier"] for e in fe["expansions"] if e["kind"] == "named_barrier"] == want["named_barrier"]
    assert [e["counter"] for e in fe["expansions"] if e["kind"] == "counter"] == want["counter"]


# ---------------------------------------------------------------- examples/hopper-gemm-split
HOPPER = json.loads((Path(__file__).parent / "golden" / "reference_hopper_gemm_split.json").read_text())


@pytest.mark.parametrize("cell", sorted(HOPPER["cells"]))
def test_hopper_gemm_split_solves_as_the_reference_solves_it(cell):
    """The reference's split GEMM (load, MMA and one of three epilogue owners; Hopper device code that
    this library does not build): its manifests, emitted by its annotation pass, and the four pipeline
    descriptions of its build.py are CHECKED and SOLVED here, to the reference's ring depth, launch
    shape, register allocation, warp map, barrier arrival counts and the high-water mark of shared
    memory (tests/golden/make_reference_hopper_gemm_split.py recorded both sides of the comparison)."""
    rec = HOPPER["cells"][cell]
    manifests = [copy.deepcopy(HOPPER["manifests"][n]) for n in rec["members"]]
    doc, want = copy.deepcopy(rec["pipeline"]), rec["reference"]
    for m in manifests:
        schema.validate_manifest(m)
    schema.validate_pipeline(doc)
    fe = linker.front_end(manifests, doc["pipeline"])
    assert {h: fe["bindings"][h][0] for h in want["depths"]} == want["depths"]
    warp_map = {role: [fe["bindings"][h][0] + off, fe["bindings"][h][0] + off + warps] for role, (h, warps, off) in fe["role_warps"].items()}
    assert warp_map == want["warp_map"]
    assert 32 * sum(w for _, w, _ in fe["role_warps"].values()) == want["threads"]
    assert fe["solver"]["high_water"]["smem"] == want["dyn_smem_bytes"]
    assert fe["solver"].get("launch_regs") == want["regs_cap"]
    assert fe["params"]["total_bytes"] == want["params_total_bytes"]
    # every claim as large as the reference makes it (where inside shared memory is the solver's choice
    # among equally good layouts); barrier claims are counted in slots here and in bytes there
    mine = {iv["handle"]: (iv["hi"] - iv["lo"]) * linker.profile_scale(fe["profile"], doc["pipeline"], d)
            for d, ivs in fe["intervals"].items() for iv in ivs}
    for ivs in want["intervals"].values():
        for handle, lo, hi in ivs:
            assert mine[handle] == hi - lo, handle
    for e in fe["expansions"]:
        ch = want["channels"][e["channel"]]
        assert (e["full"]["count"], e["empty"]["count"], e["full"]["tx_bytes"]) == (ch["arrive_full"], ch["arrive_empty"], ch["tx_bytes"])


# ---------------------------------------------------------------- examples/one-epilogue-many-producers
ONE_EPILOGUE = json.loads((Path(__file__).parent / "golden" / "reference_one_epilogue_units.json").read_text())
# the reference names a route by its path through storage; this planner by what the consumer executes
ROUTE_NAMES = {"tmem>receipt>reg": "direct_receipt", "smem>load>reg": "shared_direct"}


@pytest.mark.parametrize("cell", sorted(ONE_EPILOGUE["cells"]))
def test_one_epilogue_cells_plan_and_solve_as_the_reference_does(cell, tmp_path):
    """Tensor imports end to end on the reference's documents: three owners' manifests emitted by the reference's
    annotation pass (an accumulator tile in tensor memory behind a run-time base column, or in 128-byte-swizzled
    shared memory; a row-scale vector; an epilogue importing both) and the pipeline description its example
    generates. This driver's planner must certify every connection on the route the reference's planner
    certified, and the solve must reach the reference's launch shape, parameter layout and placements; the
    adapters it generates for the connections must compile for the profile."""
    case = ONE_EPILOGUE["cells"][cell]
    manifests = [copy.deepcopy(ONE_EPILOGUE["units"][n]["manifest"]) for n in case["units"]]
    for m in manifests:
        schema.validate_manifest(m)
    schema.validate_pipeline(copy.deepcopy(case["pipeline"]))
    fe = linker.front_end(manifests, copy.deepcopy(case["pipeline"]["pipeline"]))
    want = case["reference"]
    records = {r["name"]: r for r in fe["tensor"]}
    assert sorted(records) == sorted(want["connections"])
    for name, theirs in want["connections"].items():
        assert theirs["status"] == records[name]["outcome"] == "MODEL_SAT"
        assert records[name]["route"] == ROUTE_NAMES[theirs["route"]["id"]], name
        assert records[name]["used"]["scratch_bytes"] == 0          # a direct route stages nothing
    solved = want["solved"]
    assert 32 * sum(w for _, w, _ in fe["role_warps"].values()) == solved["threads"]
    warp_map = {role: [fe["bindings"][h][0] + off, fe["bindings"][h][0] + off + warps] for role, (h, warps, off) in fe["role_warps"].items()}
    assert warp_map == solved["warp_map"]
    # this driver's dispatch kernel owns the tensor-memory allocation and keeps a 16-byte slot for its base among
    # the stages' claims; the reference's stages allocate for themselves, so its total is the claims alone
    slot = next(iv for iv in fe["intervals"]["smem"] if iv["handle"] == linker.TMEM_SLOT_HANDLE)
    assert slot["hi"] - slot["lo"] == 16
    assert fe["solver"]["high_water"]["smem"] == solved["dyn_smem_bytes"] + 16
    assert fe["params"]["total_bytes"] == solved["params"]["total_bytes"] and fe["params"]["align"] == solved["params"]["align"]
    assert [list(e) for e in fe["params"]["entries"]] == solved["params"]["entries"]
    mine = {iv["handle"]: [iv["lo"], iv["hi"]] for ivs in fe["intervals"].values() for iv in ivs}
    for ivs in solved["intervals"].values():
        for handle, lo, hi in ivs:
            assert mine[handle][1] - mine[handle][0] == hi - lo, handle
            if lo < slot["lo"]:            # what lies behind the slot sits 16 bytes further on
                assert mine[handle] == [lo, hi], handle
            else:
                assert mine[handle] == [lo + 16, hi + 16], handle
    assert sorted(e["channel"] for e in fe["expansions"]) == solved["channels"]
    # the generated adapters are CUDA this toolchain compiles
    import subprocess
    from pipelink_b200.pipec2 import jitlink, pack, tensor_plan
    unit = tmp_path / "adapters.cu"
    unit.write_text(tensor_plan.adapters_unit(fe["tensor"], {role: (lo, hi - lo) for role, (lo, hi) in warp_map.items()}))
    done = subprocess.run([jitlink.nvcc(), "-dc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", str(pack.INCLUDE),
                           "-o", str(tmp_path / "adapters.o"), str(unit)], capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-2000:]
    text = unit.read_text()
    assert ("tcgen05.ld" in text) == (cell == "tmem")
