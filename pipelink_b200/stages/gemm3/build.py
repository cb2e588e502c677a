"""Pack, link and (optionally) build the one-TU control of the three-stage MXFP8 GEMM.

Counterpart of the reference's examples/hopper-gemm-split/build.py: each owner is packed once,
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
SIG = "void(const void* params, unsigned variant)"


def _operands(direction, role):
    return {"name": "operands", "direction": direction, "owner_role": role, "space": "smem", "scope": "cta", "proxy": "async",
            "tile": {"dtype": "e4m3+ue8m0", "shape": [2, 128, 128]},
            "layout": {"encoding": "pl-layout-v2", "elem_bits": 8, "shape": [[2], [128], [128]],
                       "stride": [[16384], [128], [1]], "swizzle": {"B": 3, "M": 4, "S": 3}},
            "ring": {"depth": {"handle": "pipelink_gemm_depth"}, "stage_stride_bytes": SLOT},
            "protocol": {"kind": "mbarrier",
                         "full": {"slots": "pipelink_gemm_full", "arrive": {"count": 1, "by": "load"}, "tx_bytes": SLOT},
                         "empty": {"slots": "pipelink_gemm_empty", "arrive": {"count": 1, "by": "mma"}, "tx_bytes": 0},
                         "init": {"owner": "load", "phase": 0, "materializer": "dispatch"}, "release": "once-per-acquire"},
            "binds": {"base": "pipelink_gemm_operands", "full": "pipelink_gemm_full", "empty": "pipelink_gemm_empty"}}


def _accumulator(direction, role):
    return {"name": "accumulator", "direction": direction, "owner_role": role, "space": "tmem", "scope": "cta", "proxy": "async",
            "tile": {"dtype": "f32", "shape": [128, 128]},
            "layout": {"encoding": "pl-layout-v2", "elem_bits": 32, "lanes": [0, 128], "cols": 128},
            "ring": {"depth": {"fixed": 1}, "stage_stride_bytes": 65536},
            "protocol": {"kind": "mbarrier",
                         "full": {"slots": "pipelink_gemm_acc_ready", "arrive": {"count": 1, "by": "mma"}, "tx_bytes": 0},
                         "empty": {"slots": "pipelink_gemm_acc_empty", "arrive": {"count": 4, "by": "epilogue"}, "tx_bytes": 0},
                         "init": {"owner": "mma", "phase": 0, "materializer": "dispatch"}, "release": "once-per-acquire"},
            "binds": {"base": "pipelink_gemm_acc", "full": "pipelink_gemm_acc_ready", "empty": "pipelink_gemm_acc_empty"}}


OPERAND_CLAIMS = [
    {"domain": "smem", "handle": "pipelink_gemm_operands", "extent": {"const": 0, "per": {"pipelink_gemm_depth": SLOT}}, "align": 1024, "lifetime": "kernel"},
    {"domain": "mbarrier", "handle": "pipelink_gemm_full", "extent": {"const": 0, "per": {"pipelink_gemm_depth": 1}}, "align": 1, "lifetime": "kernel"},
    {"domain": "mbarrier", "handle": "pipelink_gemm_empty", "extent": {"const": 0, "per": {"pipelink_gemm_depth": 1}}, "align": 1, "lifetime": "kernel"},
]
ACC_CLAIMS = [
    {"domain": "tmem", "handle": "pipelink_gemm_acc", "extent": {"const": 128, "per": {}}, "align": 32, "lifetime": "kernel"},
    {"domain": "mbarrier", "handle": "pipelink_gemm_acc_ready", "extent": {"const": 1, "per": {}}, "align": 1, "lifetime": "kernel"},
    {"domain": "mbarrier", "handle": "pipelink_gemm_acc_empty", "extent": {"const": 1, "per": {}}, "align": 1, "lifetime": "kernel"},
]
SF_CLAIM = {"domain": "tmem", "handle": "pipelink_gemm_sf", "extent": {"const": 0, "per": {"pipelink_gemm_depth": 8}}, "align": 32, "lifetime": "kernel"}


def _warp(handle, n, role, align=1):
    return {"domain": "warp", "handle": handle, "extent": {"const": n, "per": {}}, "align": align, "lifetime": "kernel", "roles": [role]}


def _layout_probe(type_name: str) -> str:
    """sha256 over the parameter struct's definition in gemm3.cuh (whitespace-normalised): the
    manifest's `sha256_of_layout_probe`, which changes whenever a field, its type or order does."""
    import hashlib
    import re
    text = (HERE / "gemm3.cuh").read_text()
    m = re.search(r"struct\s+(alignas\(\d+\)\s+)?" + type_name + r"\s*\{.*?\};", text, re.S)
    if m is None:
        raise ValueError(f"{type_name} is not defined in gemm3.cuh")
    return hashlib.sha256(" ".join(m.group(0).split()).encode()).hexdigest()


def _manifest(stage_id, prefix, role, entry, warps, endpoints, claims, params, undefined):
    params = dict(params, sha256_of_layout_probe=_layout_probe(params["type"]))
    return {"pipelink_abi": json.loads(json.dumps(ABI)),
            "stage": {"id": stage_id, "version": "1.0.0", "symbol_prefix": prefix, "entry_abi": "v2",
                      "roles": {role: {"entry": entry, "warps": warps}}, "exports": {}, "entry_signature": SIG,
                      "variants": [{"key": {}, "index": 0}]},
            "endpoints": endpoints, "claims": claims,
            "topology": {"cta_group": {"fixed": 1}, "cluster": {"compiled": [1, 1, 1], "launch": {"x_multiple_of": 1, "max": [1, 1, 1]}}, "multicast": [], "persistent": False, "scheduler": "static"},
            "params": params, "hints": {},
            "symbols": {"mechanism": "declared", "defined_strong": [entry], "defined_weak": [], "undefined": {u: "function" for u in undefined}},
            "provenance": {}, "payload": {"file": "stage.o"}}


MANIFESTS = {
    "load": _manifest("gemm.load", "gemm_load_", "load", "gemm_load_role", 1, [_operands("produce", "load")],
                      [_warp("pipelink_gemm_warp_load", 1, "load"), *OPERAND_CLAIMS],
                      {"bytes": 320, "align": 64, "type": "Gemm3LoadParams"},
                      ["pipelink_gemm_depth", "pipelink_gemm_operands", "pipelink_gemm_full", "pipelink_gemm_empty"]),
    "mma": _manifest("gemm.mma", "gemm_mma_", "mma", "gemm_mma_role", 1,
                     [_operands("consume", "mma"), _accumulator("produce", "mma")],
                     [_warp("pipelink_gemm_warp_mma", 1, "mma"), *OPERAND_CLAIMS, *ACC_CLAIMS, SF_CLAIM],
                     {"bytes": 16, "align": 16, "type": "Gemm3MmaParams"},
                     ["pipelink_gemm_depth", "pipelink_gemm_operands", "pipelink_gemm_full", "pipelink_gemm_empty",
                      "pipelink_gemm_acc", "pipelink_gemm_sf", "pipelink_gemm_acc_ready", "pipelink_gemm_acc_empty", "pipelink_tmem_slot"]),
    "epilogue_bias_silu": _manifest("gemm.epilogue.bias-silu", "gemm_epilogue_bias_silu_", "epilogue",
                                    "gemm_epilogue_bias_silu_role", 4, [_accumulator("consume", "epilogue")],
                                    [_warp("pipelink_gemm_warp_epilogue", 4, "epilogue", align=4), *ACC_CLAIMS],
                                    {"bytes": 32, "align": 16, "type": "Gemm3EpilogueParams"},
                                    ["pipelink_gemm_acc", "pipelink_gemm_acc_ready", "pipelink_gemm_acc_empty", "pipelink_tmem_slot"]),
}
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
           "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(lib), str(src)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("provider build failed:\n" + proc.stderr[-3000:])
    return lib


def write_manifests():
    for name, m in MANIFESTS.items():
        (HERE / f"{name}.manifest.json").write_text(json.dumps(m, indent=1, sort_keys=True) + "\n")


def build(out: Path, depth=None, one_tu=True):
    out.mkdir(parents=True, exist_ok=True)
    write_manifests()
    stages = []
    for name, m in MANIFESTS.items():
        pkg = out / f"{name}.plink"
        packer.pack_cu(HERE / f"{name}.cu", HERE / f"{name}.manifest.json", pkg)
        stages.append({"stage_id": m["stage"]["id"], "artifact_path": f"{name}.plink"})
    spec = out / "pipeline.json"
    spec.write_text(json.dumps(pipeline_spec(stages, depth), indent=1))
    result = linker.link(spec, out / "link")
    build_provider(out)
    if one_tu:
        # same-source single translation unit: the parity denominator for the linked image
        tu = out / "link" / "generated" / "one_tu.cu"
        tu.write_text("".join(f'#include "{HERE / (n + ".cu")}"\n' for n in MANIFESTS) +
                      '#include "binding_stub.cu"\n#include "dispatch.cu"\n')
        cmd = [jitlink.nvcc(), "-cubin", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-gencode",
               "arch=compute_100a,code=sm_100a", "-I", str(tu.parent), "-o", str(out / "link" / "one_tu.cubin"), str(tu)]
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
