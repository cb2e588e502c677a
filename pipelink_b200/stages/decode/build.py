"""Pack the decode interpreter's two owners and link them.

``decode.stream`` (the producer warp) and ``decode.interpret`` (the sixteen interpreter warps) are
packed from their annotated sources; the link solves the depth of the ``weights`` ring (6 of
{6..2}: six 32 KB stages, the partial sums, the attention workspace and the instruction copy fill
the CTA's shared memory), every shared-memory and barrier base, and checks the warp tiling the
device code relies on (interpreter warps 0-15, stream warp 16). Also builds the same sources as ONE
translation unit, the control the linked image is timed against (the reference's decode gate: a
linked build within 1 % of the single-unit build). Runs without a GPU.

    python -m pipelink_b200.stages.decode.build [--out DIR]
"""
from __future__ import annotations

import argparse
import json
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

from ...pipec2 import jitlink, link as linker, pack as packer

HERE = Path(__file__).resolve().parent
ABI = {"schema": "3.0", "target": {"profile": "sm_100a", "lto_arch": "lto_100a", "toolkit": "cuda-12.9",
                                   "math": {"ftz": False, "prec_div": True, "prec_sqrt": True, "fmad": True}}}
STAGES = ("stream", "interpret")
BASE_DOMAINS = {"pipelink_dec_ring": "smem", "pipelink_dec_partial": "smem", "pipelink_dec_scratch": "smem",
                "pipelink_dec_inst": "smem", "pipelink_dec_full": "mbarrier", "pipelink_dec_empty": "mbarrier",
                "pipelink_dec_inst_ready": "mbarrier", "pipelink_dec_warp_stream": "warp",
                "pipelink_dec_warp_interpret": "warp", "pipelink_dec_named_barrier": "named_barrier"}
_manifests = None


def manifests() -> dict:
    """{stage file stem: manifest}, emitted from the units' PL_* annotations."""
    global _manifests
    if _manifests is None:
        emitted = [packer.emit_manifest(HERE / f"{n}.cu") for n in STAGES]
        for m in emitted:
            m["pipelink_abi"] = json.loads(json.dumps(ABI))
        _manifests = dict(zip(STAGES, emitted))
    return _manifests


def pipeline_spec(stages, depth=None, values=(6, 5, 4, 3, 2)):
    handles = {"pipelink_dec_depth": {"class": "depth", "binding": "bind", "values": list(values), "owner": "channel:weights"}}
    for h, dom in BASE_DOMAINS.items():
        handles[h] = {"class": "base", "binding": "bind", "domain": dom, "owner": f"claim:{h}"}
    # the interpreter's code takes threadIdx.x as its thread index: its warps come first
    forced = {"pipelink_dec_warp_interpret": 0, "pipelink_dec_warp_stream": 16}
    if depth is not None:
        forced["pipelink_dec_depth"] = depth
    return {"pipelink_abi": ABI,
            "pipeline": {"name": "decode-interpreter", "stages": stages, "handles": handles, "phases": ["steady"], "exclusive": [],
                         "domains": {}, "depth_priority": ["pipelink_dec_depth"], "regs_priority": [], "forced_bindings": forced,
                         "topology": {"persistent": True, "scheduler": "static"}}}


def build(out: Path, depth=None, device_link=True, one_tu=True):
    """-> LinkResult; image at out/link/pipeline.cubin, control at out/link/one_tu.cubin."""
    out.mkdir(parents=True, exist_ok=True)
    with ThreadPoolExecutor(len(STAGES)) as pool:
        list(pool.map(lambda n: packer.pack_cu(HERE / f"{n}.cu", None, out / f"{n}.plink"), STAGES))
    stages = [{"stage_id": manifests()[n]["stage"]["id"], "artifact_path": f"{n}.plink"} for n in STAGES]
    spec = out / "pipeline.json"
    spec.write_text(json.dumps(pipeline_spec(stages, depth), indent=1))
    result = linker.link(spec, out / "link", device_link=device_link)
    if one_tu and device_link:
        tu = out / "link" / "generated" / "one_tu.cu"
        tu.write_text("".join(f'#include "{HERE / (n + ".cu")}"\n' for n in STAGES) +
                      '#include "binding_stub.cu"\n#include "dispatch.cu"\n')
        cmd = [jitlink.nvcc(), "-cubin", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-gencode",
               "arch=compute_100a,code=sm_100a", "-I", str(tu.parent), "-I", str(packer.INCLUDE), "-o",
               str(out / "link" / "one_tu.cubin"), str(tu)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("one-TU control failed:\n" + proc.stderr[-3000:])
    return result


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(HERE / "out"))
    ap.add_argument("--depth", type=int, default=None)
    a = ap.parse_args()
    r = build(Path(a.out), a.depth)
    print(json.dumps({"threads": r.threads, "dyn_smem_bytes": r.dyn_smem_bytes, "observed": r.observed,
                      "bindings": {k: v[0] for k, v in r.bindings.items()}}))
