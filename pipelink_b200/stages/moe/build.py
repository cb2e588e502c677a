"""Pack the MoE grouped-GEMM owners and link their compositions.

Every package's manifest comes from the ``PL_*`` annotations in its source (``pipec2 pack`` runs
the unit's host projection). The packages: ``moe.load``, ``moe.mma``, two comm owners (``moe.comm.none``, ``moe.comm.dispatch``)
and two epilogue owners (``moe.epilogue.swiglu-mxfp8``, ``moe.epilogue.rows-bf16``). One artifact
set, three images (the reference links its MoE cells the same way from one set of packages,
campaigns/mok/README.md:80-118):

    gate_up            load + mma + comm.none     + epilogue.swiglu-mxfp8   (rows already in place)
    gate_up_dispatch   load + mma + comm.dispatch + epilogue.swiglu-mxfp8   (rows pulled in the kernel)
    down               load + mma + comm.none     + epilogue.rows-bf16      (placement or combine push)
    fwd                fwd.load + fwd.mma + comm.none     + fwd.epilogue    (both projections, one launch)
    fwd_dispatch       fwd.load + fwd.mma + comm.dispatch + fwd.epilogue    (dispatch, both projections, combine push)
    fwd_full           fwd.load + fwd.mma + comm.none     + fwd.epilogue.combine   (+ group barrier and weighted epilogue)
    fwd_full_dispatch  fwd.load + fwd.mma + comm.dispatch + fwd.epilogue.combine   (the whole forward after the schedule)

The link solves the ring depth of the ``operands`` channel, every shared-memory / barrier /
tensor-memory / counter base, the warp tiling and the two register groups. Runs without a GPU.

    python -m pipelink_b200.stages.moe.build [--out DIR]
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import subprocess
from concurrent.futures import ThreadPoolExecutor

from ...pipec2 import jitlink, link as linker, pack as packer

HERE = Path(__file__).resolve().parent
TILE, SF = 128 * 128, 512
SLOT_TX = 2 * TILE + 3 * SF               # moe::SlotTx
SLOT = SLOT_TX + 512                      # moe::SlotBytes
MAX_ROW_TILES = 4096                      # moe::MaxRowTiles
COUNTER_SLOTS = 2 * MAX_ROW_TILES + 64    # rows_ready + hidden_ready + the dispatch ticket: the images' counter workspace
ABI = {"schema": "3.0", "target": {"profile": "sm_100a", "lto_arch": "lto_100a", "toolkit": "cuda-12.9",
                                   "math": {"ftz": False, "prec_div": True, "prec_sqrt": True, "fmad": True}}}
HELPERS = ("pipelink_moe_regs_helpers", "helpers", 56)     # load + mma + comm: one warpgroup
EPILOGUE = ("pipelink_moe_regs_epilogue", "epilogue", 224)  # two warpgroups
STAGES = ("load", "mma", "comm_none", "comm_dispatch", "epilogue_swiglu", "epilogue_rows", "fwd_load", "fwd_mma", "fwd_epilogue",
          "fwd_epilogue_combine")
_manifests = None


def manifests() -> dict:
    """{stage file stem: manifest}: what each unit's PL_* annotations state, read by running the
    unit's host projection (g++, no GPU and no nvcc; the undefined-symbol list is added at pack time)."""
    global _manifests
    if _manifests is None:
        with ThreadPoolExecutor(len(STAGES)) as pool:
            emitted = list(pool.map(lambda n: packer.emit_manifest(HERE / f"{n}.cu"), STAGES))
        for m in emitted:
            m["pipelink_abi"] = json.loads(json.dumps(ABI))
        _manifests = dict(zip(STAGES, emitted))
    return _manifests


def __getattr__(name):
    if name == "MANIFESTS":
        return manifests()
    raise AttributeError(name)


COMPOSITIONS = {
    "gate_up": ["load", "mma", "comm_none", "epilogue_swiglu"],
    "gate_up_dispatch": ["load", "mma", "comm_dispatch", "epilogue_swiglu"],
    "down": ["load", "mma", "comm_none", "epilogue_rows"],
    "fwd": ["fwd_load", "fwd_mma", "comm_none", "fwd_epilogue"],
    "fwd_dispatch": ["fwd_load", "fwd_mma", "comm_dispatch", "fwd_epilogue"],
    "fwd_full": ["fwd_load", "fwd_mma", "comm_none", "fwd_epilogue_combine"],
    "fwd_full_dispatch": ["fwd_load", "fwd_mma", "comm_dispatch", "fwd_epilogue_combine"],
}
BASE_DOMAINS = {"pipelink_moe_operands": "smem", "pipelink_moe_staging": "smem", "pipelink_moe_dispatch_ring": "smem",
                "pipelink_moe_hidden_ready": "gmem_counter", "pipelink_moe_ctas_done": "gmem_counter",
                "pipelink_moe_tail_barrier": "named_barrier", "pipelink_moe_full": "mbarrier",
                "pipelink_moe_empty": "mbarrier", "pipelink_moe_acc_full": "mbarrier", "pipelink_moe_acc_empty": "mbarrier",
                "pipelink_moe_drain": "mbarrier", "pipelink_moe_acc": "tmem", "pipelink_moe_sfcols": "tmem",
                "pipelink_moe_warp_load": "warp", "pipelink_moe_warp_mma": "warp", "pipelink_moe_warp_comm": "warp",
                "pipelink_moe_warp_epilogue": "warp", "pipelink_moe_rows_ready": "gmem_counter",
                "pipelink_moe_ticket": "gmem_counter"}


def pipeline_spec(name, members, stages, depth=None, values=(6, 5, 4, 3, 2)):
    claimed = {cl["handle"] for m in members for cl in manifests()[m]["claims"]}
    handles = {"pipelink_moe_depth": {"class": "depth", "binding": "bind", "values": list(values), "owner": "channel:operands"}}
    for h, dom in BASE_DOMAINS.items():
        if h in claimed:
            handles[h] = {"class": "base", "binding": "bind", "domain": dom, "owner": f"claim:{h}"}
    for handle, group, value in (HELPERS, EPILOGUE):
        handles[handle] = {"class": "regs", "binding": "bind", "domain": "regs", "values": [value], "owner": f"reg_group:{group}"}
    return {"pipelink_abi": ABI,
            "pipeline": {"name": f"moe-{name.replace('_', '-')}", "stages": stages, "handles": handles, "phases": ["steady"],
                         "exclusive": [], "domains": {"gmem_counter": {"capacity": COUNTER_SLOTS}},
                         "depth_priority": ["pipelink_moe_depth"], "regs_priority": [EPILOGUE[0], HELPERS[0]],
                         "forced_bindings": {} if depth is None else {"pipelink_moe_depth": depth},
                         "topology": {"persistent": True, "scheduler": "static"}}}


def build(out: Path, depth=None, device_link=True, one_tu=True):
    """-> {composition: LinkResult}; images at out/<composition>/pipeline.cubin. With one_tu, also
    out/<composition>/one_tu.cubin: the same stage sources, generated stub and dispatch compiled as
    ONE translation unit by nvcc, the control a linked image is timed against (the reference's gate:
    a linked build within 1 % of the single-unit build of the same sources)."""
    out.mkdir(parents=True, exist_ok=True)
    with ThreadPoolExecutor(len(STAGES)) as pool:
        list(pool.map(lambda n: packer.pack_cu(HERE / f"{n}.cu", None, out / f"{n}.plink"), STAGES))
    results = {}
    for comp, members in COMPOSITIONS.items():
        stages = [{"stage_id": manifests()[m]["stage"]["id"], "artifact_path": f"{m}.plink"} for m in members]
        spec = out / f"{comp}.pipeline.json"
        spec.write_text(json.dumps(pipeline_spec(comp, members, stages, depth), indent=1))
        results[comp] = linker.link(spec, out / comp, device_link=device_link)
        if one_tu and device_link:
            tu = out / comp / "generated" / "one_tu.cu"
            tu.write_text("".join(f'#include "{HERE / (m + ".cu")}"\n' for m in members) +
                          '#include "binding_stub.cu"\n#include "dispatch.cu"\n')
            cmd = [jitlink.nvcc(), "-cubin", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-gencode",
                   "arch=compute_100a,code=sm_100a", "-I", str(tu.parent), "-I", str(packer.INCLUDE), "-o", str(out / comp / "one_tu.cubin"), str(tu)]
            proc = subprocess.run(cmd, capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError("one-TU control failed:\n" + proc.stderr[-3000:])
    return results


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(HERE / "out"))
    ap.add_argument("--depth", type=int, default=None)
    a = ap.parse_args()
    for comp, r in build(Path(a.out), a.depth).items():
        print(comp, json.dumps({"threads": r.threads, "dyn_smem_bytes": r.dyn_smem_bytes, "tmem_columns": r.tmem_columns,
                                "regs_cap": r.regs_cap, "cluster": r.cluster,
                                "bindings": {k: v[0] for k, v in r.bindings.items()}}))
