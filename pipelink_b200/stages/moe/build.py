"""Pack the MoE grouped-GEMM owners and link their compositions.

The packages: ``moe.load``, ``moe.mma``, two comm owners (``moe.comm.none``, ``moe.comm.dispatch``)
and two epilogue owners (``moe.epilogue.swiglu-mxfp8``, ``moe.epilogue.rows-bf16``). One artifact
set, three images (the reference links its MoE cells the same way from one set of packages,
campaigns/mok/README.md:80-118):

    gate_up            load + mma + comm.none     + epilogue.swiglu-mxfp8   (rows already in place)
    gate_up_dispatch   load + mma + comm.dispatch + epilogue.swiglu-mxfp8   (rows pulled in the kernel)
    down               load + mma + comm.none     + epilogue.rows-bf16      (placement or combine push)

The link solves the ring depth of the ``operands`` channel, every shared-memory / barrier /
tensor-memory / counter base, the warp tiling and the two register groups. Runs without a GPU.

    python -m pipelink_b200.stages.moe.build [--out DIR]
"""
from __future__ import annotations

import argparse
import hashlib
import json
import re
from pathlib import Path

import subprocess

from ...pipec2 import jitlink, link as linker, pack as packer

HERE = Path(__file__).resolve().parent
TILE, SF = 128 * 128, 512
SLOT_TX = 2 * TILE + 3 * SF               # moe::SlotTx
SLOT = SLOT_TX + 512                      # moe::SlotBytes
MAX_ROW_TILES = 4096                      # moe::MaxRowTiles
ABI = {"schema": "3.0", "target": {"profile": "sm_100a", "lto_arch": "lto_100a", "toolkit": "cuda-12.9",
                                   "math": {"ftz": False, "prec_div": True, "prec_sqrt": True, "fmad": True}}}
SIG = "void(const void* params, unsigned variant)"
TOPOLOGY = {"cta_group": {"fixed": 2}, "cluster": {"compiled": [2, 1, 1], "launch": {"x_multiple_of": 2, "max": [2, 1, 1]}},
            "multicast": [], "persistent": True, "scheduler": "static"}


def _operands(direction, role):
    """The ring both CTAs of a pair fill: A tile | B tile | three scale blocks per slot. The leader
    CTA's full barrier collects one arrival and one slot payload from each CTA of the pair."""
    return {"name": "operands", "direction": direction, "owner_role": role, "space": "smem", "scope": "cluster", "proxy": "async",
            "tile": {"dtype": "e4m3+ue8m0", "shape": [2, 128, 128]},
            "layout": {"encoding": "pl-layout-v2", "elem_bits": 8, "shape": [[2], [128], [128]],
                       "stride": [[TILE], [128], [1]], "swizzle": {"B": 3, "M": 4, "S": 3}},
            "ring": {"depth": {"handle": "pipelink_moe_depth"}, "stage_stride_bytes": SLOT, "payload_bytes": SLOT_TX},
            "protocol": {"kind": "mbarrier",
                         "full": {"slots": "pipelink_moe_full", "arrive": {"count": 2, "by": "load"}, "tx_bytes": 2 * SLOT_TX},
                         "empty": {"slots": "pipelink_moe_empty", "arrive": {"count": 1, "by": "mma"}, "tx_bytes": 0},
                         "init": {"owner": "load", "phase": 0, "materializer": "dispatch"}, "release": "once-per-acquire"},
            "binds": {"base": "pipelink_moe_operands", "full": "pipelink_moe_full", "empty": "pipelink_moe_empty"}}


def _accumulator(direction, role):
    """128 lanes x 256 fp32 columns per CTA; the leader's commit completes both CTAs' full barriers,
    and every epilogue warp of the pair arrives on the leader's empty barrier."""
    return {"name": "accumulator", "direction": direction, "owner_role": role, "space": "tmem", "scope": "cluster", "proxy": "async",
            "tile": {"dtype": "f32", "shape": [128, 256]},
            "layout": {"encoding": "pl-layout-v2", "elem_bits": 32, "lanes": [0, 128], "cols": 256},
            "ring": {"depth": {"fixed": 1}, "stage_stride_bytes": 131072},
            "protocol": {"kind": "mbarrier",
                         "full": {"slots": "pipelink_moe_acc_full", "arrive": {"count": 1, "by": "mma"}, "tx_bytes": 0},
                         "empty": {"slots": "pipelink_moe_acc_empty", "arrive": {"count": 16, "by": "epilogue"}, "tx_bytes": 0},
                         "init": {"owner": "mma", "phase": 0, "materializer": "dispatch"}, "release": "once-per-acquire"},
            "binds": {"base": "pipelink_moe_acc", "full": "pipelink_moe_acc_full", "empty": "pipelink_moe_acc_empty"}}


def _rows_ready(direction, role):
    """Per row tile, how many of its 256 rows the comm owner has put in place: a grid-scoped
    counter released with red.release.gpu and acquired by the load owner before its first TMA
    read of the tile (docs/reference/annotations.md, "Counters")."""
    return {"name": "rows_ready", "direction": direction, "owner_role": role, "space": "gmem", "scope": "grid", "proxy": "generic",
            "tile": {"dtype": "e4m3+ue8m0", "shape": [256]},
            "protocol": {"kind": "counter", "counter": {"slot": "pipelink_moe_rows_ready", "release": "red.release.gpu",
                                                        "acquire": "ld.acquire.gpu"}},
            "binds": {"slot": "pipelink_moe_rows_ready"}}


def _claim(domain, handle, const=0, per=None, align=1, **extra):
    return dict({"domain": domain, "handle": handle, "extent": {"const": const, "per": per or {}}, "align": align,
                 "lifetime": "kernel"}, **extra)


OPERAND_CLAIMS = [
    _claim("smem", "pipelink_moe_operands", per={"pipelink_moe_depth": SLOT}, align=1024),
    _claim("mbarrier", "pipelink_moe_full", per={"pipelink_moe_depth": 1}),
    _claim("mbarrier", "pipelink_moe_empty", per={"pipelink_moe_depth": 1}),
]
ACC_CLAIMS = [
    _claim("tmem", "pipelink_moe_acc", const=256, align=32),
    _claim("mbarrier", "pipelink_moe_acc_full", const=1),
    _claim("mbarrier", "pipelink_moe_acc_empty", const=1),
]
SF_CLAIM = _claim("tmem", "pipelink_moe_sfcols", per={"pipelink_moe_depth": 16}, align=32)
DRAIN_CLAIM = _claim("mbarrier", "pipelink_moe_drain", const=1, init_count=1)
STAGING_CLAIM = _claim("smem", "pipelink_moe_staging", const=8 * 2048, align=16)
COUNTER_CLAIMS = [
    _claim("gmem_counter", "pipelink_moe_rows_ready", const=MAX_ROW_TILES),
    _claim("gmem_counter", "pipelink_moe_ticket", const=1),
]


def _warp(handle, n, role, align=1):
    return dict(_claim("warp", handle, const=n, align=align), roles=[role])


def _regs(handle, group, role, value):
    return {"domain": "regs", "handle": handle, "roles": [role], "values": [value], "reg_group": group}


HELPERS = ("pipelink_moe_regs_helpers", "helpers", 56)     # load + mma + comm: one warpgroup
EPILOGUE = ("pipelink_moe_regs_epilogue", "epilogue", 224)  # two warpgroups


def _layout_probe(type_name: str) -> str:
    """sha256 over the parameter struct's definition in moe.cuh (whitespace-normalised)."""
    text = (HERE / "moe.cuh").read_text()
    m = re.search(r"struct\s+(alignas\(\d+\)\s+)?" + type_name + r"\s*\{.*?\};", text, re.S)
    if m is None:
        raise ValueError(f"{type_name} is not defined in moe.cuh")
    return hashlib.sha256(" ".join(m.group(0).split()).encode()).hexdigest()


def _manifest(stage_id, role, entry, warps, endpoints, claims, params, undefined):
    prefix = re.sub(r"[.-]", "_", stage_id) + "_"
    params = dict(params, sha256_of_layout_probe=_layout_probe(params["type"]))
    return {"pipelink_abi": json.loads(json.dumps(ABI)),
            "stage": {"id": stage_id, "version": "1.0.0", "symbol_prefix": prefix, "entry_abi": "v2",
                      "roles": {role: {"entry": entry, "warps": warps}}, "exports": {}, "entry_signature": SIG,
                      "variants": [{"key": {}, "index": 0}]},
            "endpoints": endpoints, "claims": claims, "topology": json.loads(json.dumps(TOPOLOGY)),
            "params": params, "hints": {},
            "symbols": {"mechanism": "declared", "defined_strong": [entry], "defined_weak": [],
                        "undefined": {u: "function" for u in undefined}},
            "provenance": {}, "payload": {"file": "stage.o"}}


RING = ["pipelink_moe_depth", "pipelink_moe_operands", "pipelink_moe_full", "pipelink_moe_empty"]
ACC = ["pipelink_moe_acc", "pipelink_moe_acc_full", "pipelink_moe_acc_empty", "pipelink_tmem_slot"]
MANIFESTS = {
    "load": _manifest("moe.load", "load", "moe_load_role", 1,
                      [_operands("produce", "load"), _rows_ready("consume", "load")],
                      [_warp("pipelink_moe_warp_load", 1, "load"), _regs(*HELPERS[:2], "load", HELPERS[2]), *OPERAND_CLAIMS,
                       COUNTER_CLAIMS[0]],
                      {"bytes": 576, "align": 64, "type": "MoeLoadParams"}, RING + ["pipelink_moe_rows_ready"]),
    "mma": _manifest("moe.mma", "mma", "moe_mma_role", 1,
                     [_operands("consume", "mma"), _accumulator("produce", "mma")],
                     [_warp("pipelink_moe_warp_mma", 1, "mma"), _regs(*HELPERS[:2], "mma", HELPERS[2]), *OPERAND_CLAIMS,
                      *ACC_CLAIMS, SF_CLAIM, DRAIN_CLAIM],
                     {"bytes": 48, "align": 16, "type": "MoeMmaParams"},
                     RING + ACC + ["pipelink_moe_sfcols", "pipelink_moe_drain"]),
    "comm_none": _manifest("moe.comm.none", "comm", "moe_comm_none_role", 2, [_rows_ready("produce", "comm")],
                           [_warp("pipelink_moe_warp_comm", 2, "comm"), _regs(*HELPERS[:2], "comm", HELPERS[2]),
                            COUNTER_CLAIMS[0]],
                           {"bytes": 0, "align": 16, "type": "MoeMmaParams"}, []),
    "comm_dispatch": _manifest("moe.comm.dispatch", "comm", "moe_comm_dispatch_role", 2, [_rows_ready("produce", "comm")],
                               [_warp("pipelink_moe_warp_comm", 2, "comm"), _regs(*HELPERS[:2], "comm", HELPERS[2]),
                                STAGING_CLAIM, *COUNTER_CLAIMS],
                               {"bytes": 112, "align": 16, "type": "MoeCommParams"},
                               ["pipelink_moe_warp_comm", "pipelink_moe_staging", "pipelink_moe_rows_ready", "pipelink_moe_ticket"]),
    "epilogue_swiglu": _manifest("moe.epilogue.swiglu-mxfp8", "epilogue", "moe_epilogue_swiglu_mxfp8_role", 8,
                                 [_accumulator("consume", "epilogue")],
                                 [_warp("pipelink_moe_warp_epilogue", 8, "epilogue", align=4),
                                  _regs(*EPILOGUE[:2], "epilogue", EPILOGUE[2]), *ACC_CLAIMS],
                                 {"bytes": 80, "align": 16, "type": "MoeSwigluParams"}, ACC + ["pipelink_moe_warp_epilogue"]),
    "epilogue_rows": _manifest("moe.epilogue.rows-bf16", "epilogue", "moe_epilogue_rows_bf16_role", 8,
                               [_accumulator("consume", "epilogue")],
                               [_warp("pipelink_moe_warp_epilogue", 8, "epilogue", align=4),
                                _regs(*EPILOGUE[:2], "epilogue", EPILOGUE[2]), *ACC_CLAIMS, STAGING_CLAIM],
                               {"bytes": 96, "align": 16, "type": "MoeRowsParams"},
                               ACC + ["pipelink_moe_warp_epilogue", "pipelink_moe_staging"]),
}
COMPOSITIONS = {
    "gate_up": ["load", "mma", "comm_none", "epilogue_swiglu"],
    "gate_up_dispatch": ["load", "mma", "comm_dispatch", "epilogue_swiglu"],
    "down": ["load", "mma", "comm_none", "epilogue_rows"],
}
BASE_DOMAINS = {"pipelink_moe_operands": "smem", "pipelink_moe_staging": "smem", "pipelink_moe_full": "mbarrier",
                "pipelink_moe_empty": "mbarrier", "pipelink_moe_acc_full": "mbarrier", "pipelink_moe_acc_empty": "mbarrier",
                "pipelink_moe_drain": "mbarrier", "pipelink_moe_acc": "tmem", "pipelink_moe_sfcols": "tmem",
                "pipelink_moe_warp_load": "warp", "pipelink_moe_warp_mma": "warp", "pipelink_moe_warp_comm": "warp",
                "pipelink_moe_warp_epilogue": "warp", "pipelink_moe_rows_ready": "gmem_counter",
                "pipelink_moe_ticket": "gmem_counter"}


def pipeline_spec(name, members, stages, depth=None, values=(6, 5, 4, 3, 2)):
    claimed = {cl["handle"] for m in members for cl in MANIFESTS[m]["claims"]}
    handles = {"pipelink_moe_depth": {"class": "depth", "binding": "bind", "values": list(values), "owner": "channel:operands"}}
    for h, dom in BASE_DOMAINS.items():
        if h in claimed:
            handles[h] = {"class": "base", "binding": "bind", "domain": dom, "owner": f"claim:{h}"}
    for handle, group, value in (HELPERS, EPILOGUE):
        handles[handle] = {"class": "regs", "binding": "bind", "domain": "regs", "values": [value], "owner": f"reg_group:{group}"}
    return {"pipelink_abi": ABI,
            "pipeline": {"name": f"moe-{name.replace('_', '-')}", "stages": stages, "handles": handles, "phases": ["steady"],
                         "exclusive": [], "domains": {"gmem_counter": {"capacity": MAX_ROW_TILES + 64}},
                         "depth_priority": ["pipelink_moe_depth"], "regs_priority": [EPILOGUE[0], HELPERS[0]],
                         "forced_bindings": {} if depth is None else {"pipelink_moe_depth": depth},
                         "topology": {"persistent": True, "scheduler": "static"}}}


def write_manifests():
    for name, m in MANIFESTS.items():
        (HERE / f"{name}.manifest.json").write_text(json.dumps(m, indent=1, sort_keys=True) + "\n")


def build(out: Path, depth=None, device_link=True, one_tu=True):
    """-> {composition: LinkResult}; images at out/<composition>/pipeline.cubin. With one_tu, also
    out/<composition>/one_tu.cubin: the same stage sources, generated stub and dispatch compiled as
    ONE translation unit by nvcc, the control a linked image is timed against (the reference's gate:
    a linked build within 1 % of the single-unit build of the same sources)."""
    out.mkdir(parents=True, exist_ok=True)
    write_manifests()
    for name in MANIFESTS:
        packer.pack_cu(HERE / f"{name}.cu", HERE / f"{name}.manifest.json", out / f"{name}.plink")
    results = {}
    for comp, members in COMPOSITIONS.items():
        stages = [{"stage_id": MANIFESTS[m]["stage"]["id"], "artifact_path": f"{m}.plink"} for m in members]
        spec = out / f"{comp}.pipeline.json"
        spec.write_text(json.dumps(pipeline_spec(comp, members, stages, depth), indent=1))
        results[comp] = linker.link(spec, out / comp, device_link=device_link)
        if one_tu and device_link:
            tu = out / comp / "generated" / "one_tu.cu"
            tu.write_text("".join(f'#include "{HERE / (m + ".cu")}"\n' for m in members) +
                          '#include "binding_stub.cu"\n#include "dispatch.cu"\n')
            cmd = [jitlink.nvcc(), "-cubin", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-gencode",
                   "arch=compute_100a,code=sm_100a", "-I", str(tu.parent), "-o", str(out / comp / "one_tu.cubin"), str(tu)]
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
