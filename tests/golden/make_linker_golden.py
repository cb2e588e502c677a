"""Records what the REFERENCE's linker front end (schema -> pairing -> canonical layouts ->
protocol expansion -> Z3 solve) answers for this repo's three-stage GEMM packages.

Run in the build container, where the reference tree is mounted (it does not travel):

    python tests/golden/make_linker_golden.py <path to a checkout of the reference>

writes tests/golden/gemm3_reference_linker.json. Two facts of this image differ from the
reference's sm_100a profile and are patched in memory before loading, nothing else is touched:
the toolkit stamp (cuda-12.9 here, cuda-13.3.0 there) and the LTO arch spelling (lto_100a / lto_100).
Interior base addresses are not recorded: the reference has no tie-break tier for them (its solver
fixes depth, per-domain high-water marks and variants, pipec/src/pipec2/solve.py:971-977), so
only those tiers, the launch shape, the warp tiling and the failing clause ids are contract.
"""
import dataclasses
import json
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
if len(sys.argv) < 2:
    raise SystemExit("usage: " + Path(__file__).name + " <path to a checkout of the reference>")
REFERENCE = Path(sys.argv[1])
sys.path.insert(0, str(REFERENCE / "pipec" / "src"))

from pipec2 import link as rlink, profile as rprofile, schema as rschema  # noqa: E402  (the reference)
from pipec2.model import PipeLinkError as RefError  # noqa: E402
from pipec2.tensor.lifetimes import resolve_lifetimes  # noqa: E402

from pipelink_b200.stages.gemm3 import build as g3  # noqa: E402
from tests.golden import linker_cases  # noqa: E402

base = rprofile.PROFILES["sm_100a"]
rprofile.PROFILES["sm_100a"] = dataclasses.replace(
    base, toolkit="cuda-12.9", lto_arch="lto_100a",
    adapter_compile=dataclasses.replace(base.adapter_compile, toolkit="cuda-12.9"))


def front_end(pipeline, stages):
    profile = rlink.get_profile(pipeline.target.profile)
    pipeline, stages = rlink._params_composition(pipeline, stages)
    lifetimes = resolve_lifetimes(pipeline, stages)
    if lifetimes.failures:
        raise RefError(lifetimes.failures)
    pairs = rlink._pair_channels(stages)
    canon = rlink._canonical_endpoints(stages, pipeline, profile)
    rlink._unify_pairs(pairs, canon)
    expansions = sorted((rlink._expand_protocol(ch, pr, co, stages, pipeline, canon, profile) for ch, pr, co in pairs),
                        key=lambda e: e.channel)
    return rlink._solve_pipeline(pipeline, stages, canon, expansions, profile, lifetimes.ordered_pairs)


def record(solution):
    hw = {}
    for domain, ivs in solution.intervals.items():
        hw[domain] = max(iv.hi for iv in ivs)
    return {"depths": dict(solution.depths), "threads": solution.launch.threads, "regs_cap": solution.launch.regs_cap,
            "dyn_smem_bytes": solution.launch.dyn_smem_bytes, "cluster": list(solution.launch.cluster),
            "high_water": hw, "warp_map": {k: list(v) for k, v in solution.warp_map.items()},
            "extents": {iv.handle: iv.hi - iv.lo for ivs in solution.intervals.values() for iv in ivs}}


out = {"reference_profile": "sm_100a (toolkit and lto_arch stamps patched to this image's)", "solutions": {}, "negative": {}}
with tempfile.TemporaryDirectory() as tmp:
    tmp = Path(tmp)
    g3.build(tmp, one_tu=False)          # packs the three stages with this repo's packer
    stage_list = json.loads((tmp / "pipeline.json").read_text())["pipeline"]["stages"]
    for name, kwargs in linker_cases.SOLVE_CASES.items():
        spec = tmp / f"{name}.json"
        spec.write_text(json.dumps(g3.pipeline_spec(stage_list, **kwargs)))
        pipeline, artifacts = rlink._load_assembly(spec)      # reads the .plink containers
        rlink._check_symbols(artifacts)
        try:
            out["solutions"][name] = record(front_end(pipeline, [a.stage for a in artifacts]))
        except RefError as e:
            out["solutions"][name] = {"failures": sorted({f.clause_id for f in e.failures})}
    pipeline_obj = g3.pipeline_spec(stage_list)
    for name in linker_cases.NEGATIVE_CASES:
        ms = linker_cases.mutated(g3.MANIFESTS, name)
        for m in ms:   # what the packer would stamp
            m["provenance"] = {"mechanism": "declared-json", "inputs": {}}
        try:
            stages = [rschema.load_stage_manifest(m) for m in ms]
            front_end(rschema.load_pipeline(pipeline_obj), stages)
            out["negative"][name] = []
        except RefError as e:
            out["negative"][name] = sorted({f.clause_id for f in e.failures})
            print(name, [(f.clause_id, f.path, f.message) for f in e.failures][:3])

target = Path(__file__).with_name("gemm3_reference_linker.json")
target.write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
print(target, json.dumps(out["solutions"], indent=1)[:1500])
print(json.dumps(out["negative"], indent=1))
