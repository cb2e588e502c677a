"""Pack the two hello stages and link them: the smallest image with a call channel.

``hello.provider`` has no role and no params; it exports ``hello_scale``. ``hello.caller`` owns a
four-warp grid-stride loop and calls ``pipelink_call_scale``, a trampoline the LINK generates from
the two ends' declarations (same export, same C signature) into the binding stub; the LTO link
inlines it. Also builds the same sources as ONE translation unit, the control the linked image is
compared with. The reference's first tutorial builds the same pair
(examples/hello-callable/build.py). Runs without a GPU.

    python -m pipelink_b200.stages.hello.build [--out DIR]
"""
from __future__ import annotations

import argparse
import json
import subprocess
from pathlib import Path

from ...pipec2 import jitlink, link as linker, pack as packer

HERE = Path(__file__).resolve().parent
ABI = {"schema": "3.0", "target": {"profile": "sm_100a", "lto_arch": "lto_100a", "toolkit": "cuda-12.9",
                                   "math": {"ftz": False, "prec_div": True, "prec_sqrt": True, "fmad": True}}}
STAGES = ("provider", "caller")
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


def pipeline_spec(stages):
    return {"pipelink_abi": ABI,
            # the caller's role claims its warps under the handle the annotation pass derives for it
            "pipeline": {"name": "hello-callable", "stages": stages,
                         "handles": {"pipelink_call_warps": {"class": "base", "binding": "bind", "domain": "warp", "owner": "claim:call"}},
                         "phases": ["steady"], "exclusive": [],
                         "domains": {}, "depth_priority": [], "regs_priority": [], "forced_bindings": {},
                         "topology": {"persistent": False, "scheduler": "static"}}}


def build(out: Path, device_link=True, one_tu=True):
    """-> LinkResult; image at out/link/pipeline.cubin, control at out/link/one_tu.cubin."""
    out.mkdir(parents=True, exist_ok=True)
    for n in STAGES:
        packer.pack_cu(HERE / f"{n}.cu", None, out / f"{n}.plink")
    stages = [{"stage_id": manifests()[n]["stage"]["id"], "artifact_path": f"{n}.plink"} for n in STAGES]
    spec = out / "pipeline.json"
    spec.write_text(json.dumps(pipeline_spec(stages), indent=1))
    result = linker.link(spec, out / "link", device_link=device_link)
    if one_tu and device_link:
        tu = out / "link" / "generated" / "one_tu.cu"
        tu.write_text("".join(f'#include "{HERE / (n + ".cu")}"\n' for n in STAGES) +
                      '#include "binding_stub.cu"\n#include "dispatch.cu"\n')
        cmd = [jitlink.nvcc(), "-cubin", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
               "-I", str(tu.parent), "-I", str(packer.INCLUDE), "-o", str(out / "link" / "one_tu.cubin"), str(tu)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("one-TU control failed:\n" + proc.stderr[-3000:])
    return result


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(HERE / "out"))
    a = ap.parse_args()
    r = build(Path(a.out))
    print(json.dumps({"threads": r.threads, "dyn_smem_bytes": r.dyn_smem_bytes, "observed": r.observed}))
