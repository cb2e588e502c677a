"""Records what the reference's OWN annotation pass emits for the stage sources of its
`examples/one-epilogue-many-producers` that make up the two sm_100a cells of its build.py: the epilogue that
imports an accumulator tile and a row-scale vector (consumer/epilogue.cu), the provider that exports the row
scales from shared memory (providers/rowscale/rowscale.cu) and the accumulator provider
(providers/accumulator/producer_source.cu) packed twice, exporting the tile from tensor memory
(-DPL_EXPORT_TMEM) and from swizzled shared memory (-DPL_EXPORT_SMEM); its mainloop includes CUTLASS, which the
example takes from a submodule that is not checked out: pass any recent CUTLASS include tree. A smaller
tensor-memory provider (producer_m128.cu) is recorded as well. These are the units that use the tensor
annotations (PL_SITE, PL_IMPORT_TENSOR, PL_EXPORT_TENSOR, PL_BINDING): maps written as C++ lambdas, tabulated
by the pass and fitted to expressions.

It then composes the example's two sm_100a cells (accumulator provider, row-scale provider, epilogue; the
pipeline description as the example's pipelines/generate.py writes it: one base handle per claim, one
connection per export whose identity an import restates) and records what the reference's OWN tensor planner
(link._plan_tensors) decides for each connection: the status and the route it certifies.

Run in the build container, where the reference tree is mounted (it does not travel):

    python tests/golden/make_reference_one_epilogue.py <path to a checkout of the reference> <CUTLASS include dir>

writes tests/golden/reference_one_epilogue_units.json.
"""
import json
import os
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
if len(sys.argv) < 3:
    raise SystemExit("usage: " + Path(__file__).name + " <path to a checkout of the reference> <CUTLASS include dir>")
REFERENCE, CUTLASS = Path(sys.argv[1]), Path(sys.argv[2])
sys.path.insert(0, str(REFERENCE / "pipec" / "src"))
os.environ.setdefault("PIPEC_CUDA", "/usr/local/cuda")

from pipec2 import link as rlink, schema as rschema, symbols  # noqa: E402  (the reference)
from pipec2.pack.assemble import assemble  # noqa: E402
from pipec2.pack.emit import compile_registry  # noqa: E402
from pipec2.tensor.lifetimes import resolve_lifetimes  # noqa: E402

PROFILE, TOOLKIT = "sm_100a", "cuda-13.3.0"
EXAMPLE = REFERENCE / "examples" / "one-epilogue-many-producers"
TCGEN05 = {"PL_TILE_N": "128", "PL_MMA_M": "128"}          # the defines of the example's params.py for this profile
UNITS = {"consumer": ("consumer/epilogue.cu", {}), "rowscale": ("providers/rowscale/rowscale.cu", {}),
         "producer_m128": ("providers/accumulator/producer_m128.cu", {}),
         "acc_tmem": ("providers/accumulator/producer_source.cu", {**TCGEN05, "PL_EXPORT_TMEM": "1"}),
         "acc_smem": ("providers/accumulator/producer_source.cu", {**TCGEN05, "PL_EXPORT_SMEM": "1"}),
         # the Hopper provider that exports the accumulator from the warpgroup-MMA register fragment: only its host
         # projection is compiled; its placement is a bit permutation of (m, n), printed as integer bit fields
         "sm90_reg": ("providers/accumulator/producer_sm90.cu", {"PL_TILE_N": "128"}, "sm_90a")}


def emit(source: Path, defines: dict, profile: str = PROFILE) -> dict:
    env = os.environ.copy()
    cuda = symbols.cuda_home(env)
    env["PATH"] = str(cuda / "bin") + os.pathsep + env.get("PATH", "")
    env["CUDA_VISIBLE_DEVICES"] = ""
    with tempfile.TemporaryDirectory() as tmp:
        comp = compile_registry(source, Path(tmp), includes=(CUTLASS,), defines=tuple(f"{k}={v}" for k, v in defines.items()), nvcc_flags=(), profile=profile,
                                toolkit=TOOLKIT, env=env)
        return assemble(comp.registry, profile=profile, toolkit=TOOLKIT, provenance_inputs=comp.provenance_inputs,
                        math=comp.math)


record = {"units": {}}
for name, (rel, defines, *rest) in UNITS.items():
    profile = rest[0] if rest else PROFILE
    record["units"][name] = {"source": "examples/one-epilogue-many-producers/" + rel, "defines": defines, "profile": profile,
                             "manifest": emit(EXAMPLE / rel, defines, profile)}


def cell_document(cell: str, owners: list) -> dict:
    handles = {}
    for owner in owners:
        for claim in owner["claims"]:
            handles[claim["handle"]] = {"class": "base", "binding": "bind", "domain": claim["domain"], "owner": f"claim:{claim['handle']}"}
    accumulator, scale, consumer = owners
    connections = []
    for name, provider in (("acc", accumulator), ("scale", scale)):
        export, = provider["tensor"]["exports"]
        imp, = (item for item in consumer["tensor"]["imports"] if item["identity"] == export["identity"])
        connections.append({"name": name, "export": f"{provider['stage']['id']}:{export['name']}",
                            "import": f"{consumer['stage']['id']}:{imp['name']}"})
    return {"pipelink_abi": json.loads(json.dumps(accumulator["pipelink_abi"])), "pipeline": {
        "name": f"pipelink.one_epilogue.{cell}",
        "stages": [{"stage_id": o["stage"]["id"], "artifact_path": f"{o['stage']['id']}.plink"} for o in owners],
        "handles": handles, "phases": ["tensor_work"], "exclusive": [], "domains": {}, "depth_priority": [], "regs_priority": [],
        "forced_bindings": {}, "topology": {"persistent": False, "scheduler": "static"}, "tensor_connections": connections}}


record["cells"] = {}
for cell, provider in (("tmem", "acc_tmem"), ("smem", "acc_smem")):
    names = [provider, "rowscale", "consumer"]
    owners = [record["units"][n]["manifest"] for n in names]
    document = cell_document(cell, owners)
    pipe = rschema.load_pipeline(document)
    stages = [rschema.load_stage_manifest(m) for m in owners]
    profile = rlink.get_profile(pipe.target.profile)
    planned, plans = rlink._plan_tensors(pipe, stages, profile)
    routes = {plan["name"]: {"status": plan["status"], "route": plan["bounds"][plan["selected"]]["scope"]["route"]} for plan in plans}
    # and the rest of the reference's link front end, in its order (pipec/src/pipec2/link.py:1649-1690): what the
    # planned connections reserve is composed into the stages, then pairing, expansion, parameter layout and the solve
    pipe, stages = rlink._tensor_composition(pipe, stages, planned)
    pipe, stages = rlink._params_composition(pipe, stages)
    lifetimes = resolve_lifetimes(pipe, stages)
    assert not lifetimes.failures, lifetimes.failures
    pairs = rlink._pair_channels(stages)
    canon = rlink._canonical_endpoints(stages, pipe, profile)
    rlink._unify_pairs(pairs, canon)
    expansions = sorted((rlink._expand_protocol(ch, pr, co, stages, pipe, canon, profile) for ch, pr, co in pairs),
                        key=lambda e: e.channel)
    layout = rlink._params_layout(stages, profile)
    solution = rlink._solve_pipeline(pipe, stages, canon, expansions, profile, lifetimes.ordered_pairs)
    solved = {"threads": solution.launch.threads, "dyn_smem_bytes": solution.launch.dyn_smem_bytes,
              "warp_map": {k: list(v) for k, v in solution.warp_map.items()},
              "intervals": {d: sorted([iv.handle, iv.lo, iv.hi] for iv in ivs) for d, ivs in solution.intervals.items()},
              "params": {"total_bytes": layout.total_bytes, "align": layout.align, "entries": [list(e) for e in layout.entries]},
              "channels": sorted(e.channel for e in expansions)}
    record["cells"][cell] = {"units": names, "pipeline": document, "reference": {"connections": routes, "solved": solved}}
    print(cell, json.dumps(record["cells"][cell]["reference"])[:1500])

out = ROOT / "tests" / "golden" / "reference_one_epilogue_units.json"
out.write_text(json.dumps(record, indent=None, sort_keys=True) + "\n")
print(out, out.stat().st_size, "bytes")
