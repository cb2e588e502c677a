"""Records the reference's `examples/ring-pipeline` as data: the two stage manifests its OWN
annotation pass emits from its sources (pack/emit + pack/assemble, run here unmodified, without
the object-fact step that needs its pinned toolkit), the pipeline descriptions its build.py writes
(ring depth forced to 2 and to 4, and left to the solver), and what the reference's link front end
solves for each: depth, launch shape, warp map, per-domain high-water marks.

Run in the build container, where the reference tree is mounted (it does not travel):

    python tests/golden/make_reference_examples.py <path to a checkout of the reference>

writes tests/golden/reference_ring_pipeline.json.
"""
import json
import os
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
if len(sys.argv) < 2:
    raise SystemExit("usage: " + Path(__file__).name + " <path to a checkout of the reference>")
REFERENCE = Path(sys.argv[1])
sys.path.insert(0, str(REFERENCE / "pipec" / "src"))
os.environ.setdefault("PIPEC_CUDA", "/usr/local/cuda")

from pipec2 import link as rlink, schema as rschema, symbols  # noqa: E402  (the reference)
from pipec2.model import PipeLinkError as RefError  # noqa: E402
from pipec2.pack.assemble import assemble  # noqa: E402
from pipec2.pack.emit import compile_registry  # noqa: E402
from pipec2.tensor.lifetimes import resolve_lifetimes  # noqa: E402

PROFILE, TOOLKIT = "sm_100a", "cuda-13.3.0"


def emit(source: Path) -> dict:
    env = os.environ.copy()
    cuda = symbols.cuda_home(env)
    env["PATH"] = str(cuda / "bin") + os.pathsep + env.get("PATH", "")
    env["CUDA_VISIBLE_DEVICES"] = ""
    with tempfile.TemporaryDirectory() as d:
        comp = compile_registry(source, Path(d), includes=(), defines=(), nvcc_flags=(), profile=PROFILE, toolkit=TOOLKIT, env=env)
        return assemble(comp.registry, profile=PROFILE, toolkit=TOOLKIT, provenance_inputs=comp.provenance_inputs, math=comp.math)


def pipeline(abi, stages, depth):
    """examples/ring-pipeline/build.py:pipeline, restated as data."""
    handles = {"pipelink_ring_depth": {"class": "depth", "binding": "bind", "values": [2, 4], "owner": "channel:tile_ring"}}
    for name, domain in (("base", "smem"), ("full", "mbarrier"), ("empty", "mbarrier"), ("warp_producer", "warp"),
                         ("warp_consumer", "warp")):
        handle = f"pipelink_ring_{name}"
        handles[handle] = {"class": "base", "binding": "bind", "domain": domain, "owner": f"claim:{handle}"}
    return {"pipelink_abi": abi,
            "pipeline": {"name": f"ring-pipeline-depth-{depth}", "stages": stages, "handles": handles, "phases": ["steady"],
                         "exclusive": [], "domains": {}, "depth_priority": ["pipelink_ring_depth"], "regs_priority": [],
                         "forced_bindings": {} if depth is None else {"pipelink_ring_depth": depth},
                         "topology": {"persistent": False, "scheduler": "static"}}}


def front_end(pipe, stages):
    profile = rlink.get_profile(pipe.target.profile)
    pipe, stages = rlink._params_composition(pipe, stages)
    lifetimes = resolve_lifetimes(pipe, stages)
    if lifetimes.failures:
        raise RefError(lifetimes.failures)
    pairs = rlink._pair_channels(stages)
    canon = rlink._canonical_endpoints(stages, pipe, profile)
    rlink._unify_pairs(pairs, canon)
    expansions = sorted((rlink._expand_protocol(ch, pr, co, stages, pipe, canon, profile) for ch, pr, co in pairs),
                        key=lambda e: e.channel)
    return rlink._solve_pipeline(pipe, stages, canon, expansions, profile, lifetimes.ordered_pairs), expansions


def record(solution, expansions):
    hw = {domain: max(iv.hi for iv in ivs) for domain, ivs in solution.intervals.items()}
    exp = expansions[0]
    return {"depths": dict(solution.depths), "threads": solution.launch.threads, "dyn_smem_bytes": solution.launch.dyn_smem_bytes,
            "cluster": list(solution.launch.cluster), "high_water": hw,
            "warp_map": {k: list(v) for k, v in solution.warp_map.items()},
            "extents": {iv.handle: iv.hi - iv.lo for ivs in solution.intervals.values() for iv in ivs},
            "arrive_full": list(exp.arrive_full) if isinstance(exp.arrive_full, (list, tuple)) else exp.arrive_full,
            "arrive_empty": list(exp.arrive_empty) if isinstance(exp.arrive_empty, (list, tuple)) else exp.arrive_empty,
            "tx_bytes": exp.tx_bytes_producer}


src = REFERENCE / "examples" / "ring-pipeline" / "src"
manifests = [emit(src / "producer.cu"), emit(src / "consumer.cu")]
stage_list = [{"stage_id": m["stage"]["id"], "artifact_path": f"{m['stage']['id']}.plink"} for m in manifests]
out = {"source": "examples/ring-pipeline (src/producer.cu, src/consumer.cu, build.py)", "manifests": manifests, "pipelines": {},
       "reference": {}}
for name, depth in (("depth-2", 2), ("depth-4", 4), ("solved", None)):
    doc = pipeline(manifests[0]["pipelink_abi"], stage_list, depth)
    out["pipelines"][name] = doc
    stages = [rschema.load_stage_manifest(m) for m in manifests]
    solution, expansions = front_end(rschema.load_pipeline(doc), stages)
    out["reference"][name] = record(solution, expansions)
dst = ROOT / "tests" / "golden" / "reference_ring_pipeline.json"
dst.write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
print(dst, json.dumps(out["reference"], indent=1))
