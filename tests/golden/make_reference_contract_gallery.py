"""Records the reference's `examples/contract-gallery` as data: the T2 ring producer's manifest and
the manifests its OWN annotation pass emits for the original consumer, the square replacement and
the six intentionally wrong consumers (`consumers/*.cu`), each with what the REFERENCE does with it
here: the clause its pack step or its link front end raises, or the solved launch shape.

Run in the build container, where the reference tree is mounted (it does not travel):

    python tests/golden/make_reference_contract_gallery.py <path to a checkout of the reference>

writes tests/golden/reference_contract_gallery.json, and tests/golden/reference_hello_callable.json: the
two manifests of `examples/hello-callable` (a role-less provider and a caller joined by a call channel),
the pipeline description its build.py writes, and the launch shape and parameter layout the reference's
front end derives.
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
RING = REFERENCE / "examples" / "ring-pipeline"
GALLERY = REFERENCE / "examples" / "contract-gallery" / "consumers"
# examples/contract-gallery/check.py:CASES, with the clause its table expects
CASES = (("baseline", RING / "src" / "consumer.cu", None), ("protocol", GALLERY / "protocol.cu", "L-PROTO"),
         ("topology", GALLERY / "topology.cu", "L-TOPO"), ("handle", GALLERY / "handle.cu", "L-HANDLE"),
         ("init", GALLERY / "init.cu", "P-INIT"), ("params", GALLERY / "params.cu", "L-PARAMS"),
         ("phase", GALLERY / "phase.cu", "L-PHASE"), ("swap", GALLERY / "swap.cu", None))


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
                         "forced_bindings": {"pipelink_ring_depth": depth},
                         "topology": {"persistent": False, "scheduler": "static"}}}


def front_end(pipe, stages):
    """The phases of the reference's link() before code generation, in its order
    (pipec/src/pipec2/link.py:98-140, 1614-1700), on loaded documents."""
    profile = rlink.get_profile(pipe.target.profile)
    stages, _dropped = rlink._prune_unreferenced_exports(stages)
    failures = rschema.validate_assembly(pipe, stages)
    if failures:
        raise RefError(failures)
    pipe, stages = rlink._params_composition(pipe, stages)
    lifetimes = resolve_lifetimes(pipe, stages)
    if lifetimes.failures:
        raise RefError(lifetimes.failures)
    pairs = rlink._pair_channels(stages)
    canon = rlink._canonical_endpoints(stages, pipe, profile)
    rlink._unify_pairs(pairs, canon)
    expansions = sorted((rlink._expand_protocol(ch, pr, co, stages, pipe, canon, profile) for ch, pr, co in pairs),
                        key=lambda e: e.channel)
    rlink._params_layout(stages, profile)
    return rlink._solve_pipeline(pipe, stages, canon, expansions, profile, lifetimes.ordered_pairs)


def failure_record(err):
    return [{"clause": f.clause_id, "path": f.path} for f in err.failures]


producer = emit(RING / "src" / "producer.cu")
out = {"source": "examples/contract-gallery (check.py:CASES, consumers/*.cu) over examples/ring-pipeline/src/producer.cu",
       "producer": producer, "cases": {}}
for name, source, expected in CASES:
    case = {"expected_clause": expected, "source": str(source.relative_to(REFERENCE))}
    try:
        consumer = emit(source)
    except RefError as err:
        case.update(phase="pack", reference=failure_record(err), manifest=None)
        out["cases"][name] = case
        continue
    case["manifest"] = consumer
    stage_list = [{"stage_id": producer["stage"]["id"], "artifact_path": "producer.plink"},
                  {"stage_id": consumer["stage"]["id"], "artifact_path": f"{name}.plink"}]
    doc = pipeline(producer["pipelink_abi"], stage_list, 2)
    case["pipeline"] = doc
    try:
        stages = [rschema.load_stage_manifest(m) for m in (producer, consumer)]
        solution = front_end(rschema.load_pipeline(doc), stages)
        case.update(phase="link", reference="OK", launch={"threads": solution.launch.threads, "dyn_smem_bytes": solution.launch.dyn_smem_bytes})
    except RefError as err:
        case.update(phase="link", reference=failure_record(err))
    out["cases"][name] = case
dst = ROOT / "tests" / "golden" / "reference_contract_gallery.json"
dst.write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
print(dst)
for name, case in out["cases"].items():
    print(name, case["expected_clause"], case["phase"], case["reference"], case.get("launch"))


# ---------------------------------------------------------------- examples/hello-callable
HELLO = REFERENCE / "examples" / "hello-callable" / "src"
hello = [emit(HELLO / "provider.cu"), emit(HELLO / "caller.cu")]
hello_doc = {"pipelink_abi": hello[1]["pipelink_abi"],
             "pipeline": {"name": "hello-callable",       # examples/hello-callable/build.py:56-70, restated as data
                          "stages": [{"stage_id": m["stage"]["id"], "artifact_path": f"{n}.plink"} for m, n in zip(hello, ("provider", "caller"))],
                          "handles": {"pipelink_call_warps": {"class": "base", "binding": "bind", "domain": "warp", "owner": "claim:call"}},
                          "phases": ["call"], "exclusive": [], "domains": {}, "depth_priority": [], "regs_priority": [],
                          "forced_bindings": {}, "topology": {"persistent": False, "scheduler": "static"}}}
hello_stages = [rschema.load_stage_manifest(m) for m in hello]
hello_pipe = rschema.load_pipeline(hello_doc)
solution = front_end(hello_pipe, hello_stages)
layout = rlink._params_layout(hello_stages, rlink.get_profile(hello_pipe.target.profile))
record = {"source": "examples/hello-callable (src/provider.cu, src/caller.cu, build.py)", "manifests": hello, "pipeline": hello_doc,
          "reference": {"threads": solution.launch.threads, "dyn_smem_bytes": solution.launch.dyn_smem_bytes,
                        "warp_map": {k: list(v) for k, v in solution.warp_map.items()},
                        "params": {"total_bytes": layout.total_bytes, "entries": [list(e) for e in layout.entries]}}}
dst = ROOT / "tests" / "golden" / "reference_hello_callable.json"
dst.write_text(json.dumps(record, indent=1, sort_keys=True) + "\n")
print(dst, json.dumps(record["reference"]))
