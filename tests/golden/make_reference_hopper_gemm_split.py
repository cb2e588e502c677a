"""Records the reference's `examples/hopper-gemm-split` as data: the five stage manifests its OWN
annotation pass emits for profile sm_90a (load, MMA and three epilogue owners; only the host
projection of the sources is compiled, so no Hopper device code is built), the four pipeline
descriptions its build.py writes (store, bias_relu and rowscale epilogues at ring depth 4, store at
depth 2), and what the reference's link front end solves for each.

The example's sources include CUTLASS headers from a submodule that is not checked out in the
reference tree; pass a CUTLASS include directory (any recent one: only declarations are needed):

    python tests/golden/make_reference_hopper_gemm_split.py <path to a checkout of the reference> <cutlass include dir>

writes tests/golden/reference_hopper_gemm_split.json.
"""
import json
import os
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
if len(sys.argv) < 3:
    raise SystemExit("usage: " + Path(__file__).name + " <path to a checkout of the reference> <cutlass include dir>")
REFERENCE, CUTLASS = Path(sys.argv[1]), Path(sys.argv[2])
sys.path.insert(0, str(REFERENCE / "pipec" / "src"))
os.environ.setdefault("PIPEC_CUDA", "/usr/local/cuda")

from pipec2 import link as rlink, schema as rschema, symbols  # noqa: E402  (the reference)
from pipec2.pack.assemble import assemble  # noqa: E402
from pipec2.pack.emit import compile_registry  # noqa: E402
from pipec2.tensor.lifetimes import resolve_lifetimes  # noqa: E402

PROFILE, TOOLKIT = "sm_90a", "cuda-13.3.0"
EXAMPLE = REFERENCE / "examples" / "hopper-gemm-split"
CELLS = (("store", 4), ("bias_relu", 4), ("rowscale", 4), ("store", 2))      # examples/hopper-gemm-split/build.py:19


def emit(source: Path) -> dict:
    env = os.environ.copy()
    cuda = symbols.cuda_home(env)
    env["PATH"] = str(cuda / "bin") + os.pathsep + env.get("PATH", "")
    env["CUDA_VISIBLE_DEVICES"] = ""
    with tempfile.TemporaryDirectory() as d:
        comp = compile_registry(source, Path(d), includes=(CUTLASS, EXAMPLE / "src"), defines=(), nvcc_flags=(), profile=PROFILE,
                                toolkit=TOOLKIT, env=env)
        return assemble(comp.registry, profile=PROFILE, toolkit=TOOLKIT, provenance_inputs=comp.provenance_inputs, math=comp.math)


def pipeline_spec(abi, stages, name, depth):
    """examples/hopper-gemm-split/build.py:22-63, restated as data."""
    handles = {"pipelink_gemm_depth": {"class": "depth", "binding": "bind", "values": [4, 2], "owner": "channel:operands"},
               "pipelink_launch_regs": {"class": "regs", "binding": "bind", "domain": "regs", "values": [168], "owner": "reg_group:launch"}}
    for handle, domain in (("pipelink_gemm_operands", "smem"), ("pipelink_gemm_full", "mbarrier"), ("pipelink_gemm_empty", "mbarrier"),
                           ("pipelink_gemm_output", "smem"), ("pipelink_gemm_ready", "mbarrier"), ("pipelink_gemm_drained", "mbarrier"),
                           ("pipelink_gemm_warp_load", "warp"), ("pipelink_gemm_warp_mma", "warp"), ("pipelink_gemm_warp_epilogue", "warp")):
        handles[handle] = {"class": "base", "binding": "bind", "domain": domain, "owner": f"claim:{handle}"}
    return {"pipelink_abi": abi,
            "pipeline": {"name": f"hopper-gemm-split-{name}", "stages": stages, "handles": handles, "phases": ["steady"], "exclusive": [],
                         "domains": {}, "depth_priority": ["pipelink_gemm_depth"], "regs_priority": ["pipelink_launch_regs"],
                         "forced_bindings": {"pipelink_gemm_depth": depth}, "topology": {"persistent": False, "scheduler": "static"}}}


def front_end(doc, manifests):
    pipe = rschema.load_pipeline(doc)
    stages = [rschema.load_stage_manifest(m) for m in manifests]
    profile = rlink.get_profile(pipe.target.profile)
    stages, _dropped = rlink._prune_unreferenced_exports(stages)
    failures = rschema.validate_assembly(pipe, stages)
    assert not failures, failures
    pipe, stages = rlink._params_composition(pipe, stages)
    lifetimes = resolve_lifetimes(pipe, stages)
    assert not lifetimes.failures
    pairs = rlink._pair_channels(stages)
    canon = rlink._canonical_endpoints(stages, pipe, profile)
    rlink._unify_pairs(pairs, canon)
    expansions = sorted((rlink._expand_protocol(ch, pr, co, stages, pipe, canon, profile) for ch, pr, co in pairs),
                        key=lambda e: e.channel)
    layout = rlink._params_layout(stages, profile)
    solution = rlink._solve_pipeline(pipe, stages, canon, expansions, profile, lifetimes.ordered_pairs)
    return solution, expansions, layout


names = ("load", "mma", "epilogue_store", "epilogue_bias_relu", "epilogue_rowscale")
manifests = {n: emit(EXAMPLE / "src" / f"{n}.cu") for n in names}
out = {"source": "examples/hopper-gemm-split (src/*.cu, build.py)", "manifests": manifests, "cells": {}}
for epilogue, depth in CELLS:
    cell = f"{epilogue}-d{depth}"
    members = ("load", "mma", f"epilogue_{epilogue}")
    stages = [{"stage_id": manifests[n]["stage"]["id"], "artifact_path": f"../{n}.plink"} for n in members]
    doc = pipeline_spec(manifests["load"]["pipelink_abi"], stages, cell, depth)
    solution, expansions, layout = front_end(doc, [manifests[n] for n in members])
    out["cells"][cell] = {"members": list(members), "pipeline": doc, "reference": {
        "depths": dict(solution.depths), "threads": solution.launch.threads, "dyn_smem_bytes": solution.launch.dyn_smem_bytes,
        "regs_cap": solution.launch.regs_cap, "warp_map": {k: list(v) for k, v in solution.warp_map.items()},
        "intervals": {d: sorted([iv.handle, iv.lo, iv.hi] for iv in ivs) for d, ivs in solution.intervals.items()},
        "params_total_bytes": layout.total_bytes,
        "channels": {e.channel: {"arrive_full": e.arrive_full, "arrive_empty": e.arrive_empty, "tx_bytes": e.tx_bytes_producer}
                     for e in expansions}}}
dst = ROOT / "tests" / "golden" / "reference_hopper_gemm_split.json"
dst.write_text(json.dumps(out, indent=1, sort_keys=True, default=list) + "\n")
print(dst)
for cell, rec in out["cells"].items():
    print(cell, json.dumps(rec["reference"], default=list)[:700])
