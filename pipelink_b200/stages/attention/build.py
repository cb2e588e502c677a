"""Pack the prefill attention kernel's owners and link their compositions.

Seven packages from annotated sources: two load owners (keys local / key blocks behind readiness
counters), the MMA owner, two gather owners (none / the context-parallel K/V exchange by ticket)
and two softmax owners (plain / tanh soft cap). One artifact set, three images, the way the
reference composes its attention kernel from mask, score and gather stage variants:

    prefill          load          + mma + gather.none + softmax
    prefill_softcap  load          + mma + gather.none + softmax.softcap
    prefill_cp       load.counters + mma + gather.push + softmax

The link solves the depth of the K and V rings (2: Q, two K and two V tiles of 32 KB fill the
CTA's shared memory), every shared-memory / barrier / tensor-memory base and the warp tiling
(the softmax owner on a multiple of four). Runs without a GPU.

    python -m pipelink_b200.stages.attention.build [--out DIR]
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
STAGES = ("load", "load_counters", "mma", "gather_none", "gather_push", "softmax", "softmax_softcap")
COMPOSITIONS = {
    "prefill": ["load", "mma", "gather_none", "softmax"],
    "prefill_softcap": ["load", "mma", "gather_none", "softmax_softcap"],
    "prefill_cp": ["load_counters", "mma", "gather_push", "softmax"],
}
BASE_DOMAINS = {**{f"pipelink_attn_{n}": "smem" for n in ("q", "k", "v")},
                **{f"pipelink_attn_{n}": "mbarrier" for n in ("q_full", "q_empty", "k_full", "k_empty", "v_full", "v_empty",
                                                              "s_full", "p_full", "o_full", "o_free", "drain")},
                "pipelink_attn_s": "tmem", "pipelink_attn_o": "tmem",
                **{f"pipelink_attn_warp_{n}": "warp" for n in ("load", "mma", "gather", "softmax")}}
_manifests = None


def manifests() -> dict:
    """{stage file stem: manifest}, emitted from the units' PL_* annotations."""
    global _manifests
    if _manifests is None:
        with ThreadPoolExecutor(len(STAGES)) as pool:
            emitted = list(pool.map(lambda n: packer.emit_manifest(HERE / f"{n}.cu"), STAGES))
        for m in emitted:
            m["pipelink_abi"] = json.loads(json.dumps(ABI))
        _manifests = dict(zip(STAGES, emitted))
    return _manifests


def pipeline_spec(name, stages, values=(2,)):
    handles = {"pipelink_attn_kv_depth": {"class": "depth", "binding": "bind", "values": list(values), "owner": "channel:k_tiles"}}
    for h, dom in BASE_DOMAINS.items():
        handles[h] = {"class": "base", "binding": "bind", "domain": dom, "owner": f"claim:{h}"}
    return {"pipelink_abi": ABI,
            "pipeline": {"name": f"attention-{name.replace('_', '-')}", "stages": stages, "handles": handles, "phases": ["steady"],
                         "exclusive": [], "domains": {}, "depth_priority": ["pipelink_attn_kv_depth"], "regs_priority": [],
                         "forced_bindings": {}, "topology": {"persistent": True, "scheduler": "static"}}}


def build(out: Path, device_link=True, one_tu=True):
    """-> {composition: LinkResult}; images at out/<composition>/pipeline.cubin (+ one_tu.cubin)."""
    out.mkdir(parents=True, exist_ok=True)
    with ThreadPoolExecutor(len(STAGES)) as pool:
        list(pool.map(lambda n: packer.pack_cu(HERE / f"{n}.cu", None, out / f"{n}.plink"), STAGES))
    results = {}
    for comp, members in COMPOSITIONS.items():
        stages = [{"stage_id": manifests()[m]["stage"]["id"], "artifact_path": f"{m}.plink"} for m in members]
        spec = out / f"{comp}.pipeline.json"
        spec.write_text(json.dumps(pipeline_spec(comp, stages), indent=1))
        results[comp] = linker.link(spec, out / comp, device_link=device_link)
        if one_tu and device_link:
            tu = out / comp / "generated" / "one_tu.cu"
            tu.write_text("".join(f'#include "{HERE / (m + ".cu")}"\n' for m in members) +
                          '#include "binding_stub.cu"\n#include "dispatch.cu"\n')
            cmd = [jitlink.nvcc(), "-cubin", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-gencode",
                   "arch=compute_100a,code=sm_100a", "-I", str(tu.parent), "-I", str(packer.INCLUDE), "-o",
                   str(out / comp / "one_tu.cubin"), str(tu)]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError("one-TU control failed:\n" + proc.stderr[-3000:])
    return results


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(HERE / "out"))
    a = ap.parse_args()
    for comp, r in build(Path(a.out)).items():
        print(comp, json.dumps({"threads": r.threads, "dyn_smem_bytes": r.dyn_smem_bytes, "tmem_columns": r.tmem_columns,
                                "observed": r.observed, "bindings": {k: v[0] for k, v in r.bindings.items()}}))
