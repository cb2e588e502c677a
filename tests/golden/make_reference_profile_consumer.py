"""Records the reference's `examples/profile-consumer` as data: the three stage manifests its OWN
annotation pass emits (a scheduler stage and two instruction stages that hand a shared-memory page to
each other through a named barrier and a grid-scoped counter; the pages are claims of a
pipeline-defined page domain that live in mutually exclusive phases), its pipeline description, what
the reference's link front end solves for it, and what it does with three one-line changes of the
pipeline description.

Run in the build container, where the reference tree is mounted (it does not travel):

    python tests/golden/make_reference_profile_consumer.py <path to a checkout of the reference>

writes tests/golden/reference_profile_consumer.json.
"""
import copy
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
EXAMPLE = REFERENCE / "examples" / "profile-consumer"


def emit(source: Path) -> dict:
    env = os.environ.copy()
    cuda = symbols.cuda_home(env)
    env["PATH"] = str(cuda / "bin") + os.pathsep + env.get("PATH", "")
    env["CUDA_VISIBLE_DEVICES"] = ""
    with tempfile.TemporaryDirectory() as d:
        comp = compile_registry(source, Path(d), includes=(EXAMPLE / "src", REFERENCE / "pipec/src/pipec2/host/include"), defines=(),
                                nvcc_flags=(), profile=PROFILE, toolkit=TOOLKIT, env=env)
        return assemble(comp.registry, profile=PROFILE, toolkit=TOOLKIT, provenance_inputs=comp.provenance_inputs, math=comp.math)


def front_end(doc, manifests):
    """The phases of the reference's link() before code generation, in its order
    (pipec/src/pipec2/link.py:98-140, 1614-1700), on loaded documents."""
    pipe = rschema.load_pipeline(doc)
    stages = [rschema.load_stage_manifest(m) for m in manifests]
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
    solution = rlink._solve_pipeline(pipe, stages, canon, expansions, profile, lifetimes.ordered_pairs)
    return solution, expansions


def outcome(doc, manifests):
    try:
        solution, expansions = front_end(doc, manifests)
    except RefError as err:
        return {"failures": [{"clause": f.clause_id, "path": f.path} for f in err.failures]}
    return {"threads": solution.launch.threads, "dyn_smem_bytes": solution.launch.dyn_smem_bytes,
            "warp_map": {k: list(v) for k, v in solution.warp_map.items()},
            "intervals": {d: sorted([iv.handle, iv.lo, iv.hi] for iv in ivs) for d, ivs in solution.intervals.items()},
            "named_barrier": [list(e.named_barrier) for e in expansions if e.named_barrier],
            "counter": [[e.counter[0], e.counter[1], list(e.counter[2])] for e in expansions if e.counter]}


manifests = [emit(EXAMPLE / "src" / f"{n}.cu") for n in ("interpreter", "instruction1", "instruction2")]
doc = json.loads((EXAMPLE / "manifests" / "pipeline.json").read_text())
doc["pipelink_abi"] = manifests[0]["pipelink_abi"]


def changed(edit):
    d = copy.deepcopy(doc)
    edit(d["pipeline"])
    return d


cases = {
    "as shipped": doc,
    "phases not declared exclusive": changed(lambda p: p.update(exclusive=[])),
    "second page outside the page domain": changed(lambda p: p["forced_bindings"].update(pipelink_profile_consumer_page_stage2=2)),
    "pages apart": changed(lambda p: p["forced_bindings"].update(pipelink_profile_consumer_page_stage2=0)),
    "a pattern other than instr_*": changed(lambda p: p.update(exclusive=[["instr_org*", "instr_*"]])),
}
out = {"source": "examples/profile-consumer (src/interpreter.cu, src/instruction1.cu, src/instruction2.cu, manifests/pipeline.json)",
       "manifests": manifests, "cases": {name: {"pipeline": d, "reference": outcome(d, manifests)} for name, d in cases.items()}}
dst = ROOT / "tests" / "golden" / "reference_profile_consumer.json"
dst.write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
print(dst)
for name, case in out["cases"].items():
    print(name, "->", json.dumps(case["reference"])[:400])
