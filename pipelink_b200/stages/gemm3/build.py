"""Pack, link and (optionally) build the one-TU control of the three-stage MXFP8 GEMM.

Counterpart of the reference's examples/hopper-gemm-split/build.py: each owner is packed once
(its manifest emitted from the PL_* annotations in its source),
the pipeline description declares the handles (ring depth with candidate values, resource bases),
and ``link`` solves them. Everything here runs without a GPU.

    python -m pipelink_b200.stages.gemm3.build [--out DIR] [--depth N]
"""
from __future__ import annotations

import argparse
import json
import subprocess
from pathlib import Path

from ...pipec2 import jitlink, link as linker, pack as packer
from ...pipec2.profile import PROFILES

HERE = Path(__file__).resolve().parent
SLOT = 2 * 128 * 128 + 2 * 512          # gemm3::SlotBytes
ABI = {"schema": "3.0", "target": {"profile": "sm_100a", "lto_arch": "lto_100a", "toolkit": "cuda-12.9",
                                   "math": {"ftz": False, "prec_div": True, "prec_sqrt": True, "fmad": True}}}
STAGES = ("load", "mma", "epilogue_bias_silu")
_manifests = None


def manifests() -> dict:
    """{stage file stem: manifest}: what each unit's PL_* annotations state (the unit's host projection,
    run with g++; the undefined-symbol list is added at pack time)."""
    global _manifests
    if _manifests is None:
        emitted = [packer.emit_manifest(HERE / f"{n}.cu") for n in STAGES]
        for m in emitted:
            m["pipelink_abi"] = json.loads(json.dumps(ABI))
            m["symbols"].update(mechanism="ptx-extern", defined_weak=[], undefined={})
            m["provenance"], m["payload"] = {}, {"file": "stage.o"}
        _manifests = dict(zip(STAGES, emitted))
    return _manifests


def __getattr__(name):
    if name == "MANIFESTS":
        return manifests()
    raise AttributeError(name)


BASE_HANDLES = {"pipelink_gemm_operands": "smem", "pipelink_gemm_full": "mbarrier", "pipelink_gemm_empty": "mbarrier",
                "pipelink_gemm_acc_ready": "mbarrier", "pipelink_gemm_acc_empty": "mbarrier", "pipelink_gemm_acc": "tmem", "pipelink_gemm_sf": "tmem",
                "pipelink_gemm_warp_load": "warp", "pipelink_gemm_warp_mma": "warp", "pipelink_gemm_warp_epilogue": "warp"}


def pipeline_spec(stages, depth=None, values=(6, 5, 4, 3, 2)):
    handles = {"pipelink_gemm_depth": {"class": "depth", "binding": "bind", "values": list(values), "owner": "channel:operands"}}
    for h, dom in BASE_HANDLES.items():
        handles[h] = {"class": "base", "binding": "bind", "domain": dom, "owner": f"claim:{h}"}
    return {"pipelink_abi": ABI,
            "pipeline": {"name": "mxfp8-gemm3-bias-silu", "stages": stages, "handles": handles, "phases": ["steady"],
                         "exclusive": [], "domains": {}, "depth_priority": ["pipelink_gemm_depth"], "regs_priority": [],
                         "forced_bindings": {} if depth is None else {"pipelink_gemm_depth": depth},
                         "topology": {"persistent": False, "scheduler": "static"}}}


def build_provider(out: Path) -> Path:
    """The group's params provider (host code): out/libgemm3_provider.so."""
    out.mkdir(parents=True, exist_ok=True)
    lib = out / "libgemm3_provider.so"
    src = HERE / "host" / "provider.cu"
    deps = [src, HERE / "gemm3.cuh", HERE.parents[2] / "include" / "pipelink_host_abi_v2.h"]
    if lib.exists() and all(d.stat().st_mtime <= lib.stat().st_mtime for d in deps):
        return lib
    cmd = [jitlink.nvcc(), "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "--expt-relaxed-constexpr",
           "-gencode", "arch=compute_100a,code=sm_100a", "-I", str(packer.INCLUDE), "-o", str(lib), str(src)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("provider build failed:\n" + proc.stderr[-3000:])
    return lib


def build(out: Path, depth=None, one_tu=True):
    out.mkdir(parents=True, exist_ok=True)
    stages = []
    for name, m in manifests().items():
        packer.pack_cu(HERE / f"{name}.cu", None, out / f"{name}.plink")
        stages.append({"stage_id": m["stage"]["id"], "artifact_path": f"{name}.plink"})
    spec = out / "pipeline.json"
    spec.write_text(json.dumps(pipeline_spec(stages, depth), indent=1))
    result = linker.link(spec, out / "link")
    build_provider(out)
    if one_tu:
        # same-source single translation unit: the parity denominator for the linked image
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
    print(json.dumps({"threads": r.threads, "dyn_smem_bytes": r.dyn_smem_bytes, "tmem_columns": r.tmem_columns,
                      "bindings": r.bindings}, indent=1))
