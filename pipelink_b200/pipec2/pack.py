"""``pipec2 pack``: stage source -> ``.plink``.

The manifest comes from the translation unit itself, the way the reference emits it by running the
host projection of the unit's ``PL_*`` annotations (docs/reference/pack-and-link.md:23-43,
docs/reference/annotations.md): the unit is compiled once with ``-DPIPELINK_EMIT`` as a host
program whose ``main`` (from ``<pipelink/stage.hpp>``) prints the schema-3.0 records, sizes and
member offsets of the parameter block included, and once as the LTO payload
(``nvcc -dc -gencode arch=compute_100a,code=lto_100a``). The undefined ``pipelink_*`` symbols the
link must bind are read from the unit's own PTX (``.extern .func`` declarations survive only for
functions the code calls). A unit without annotations can still be packed with a manifest kept as
JSON beside it (``manifest_path``).
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import subprocess
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

from . import container, jitlink, schema
from .model import fail
from .profile import PROFILES

INCLUDE = Path(__file__).resolve().parent / "include"
CUDA_INCLUDE = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
ABI = {"schema": "3.0", "target": {"toolkit": "cuda-12.9", "math": {"ftz": False, "prec_div": True, "prec_sqrt": True,
                                                                   "fmad": True}}}


def emit_manifest(source, includes=(), defines=(), profile="sm_100a") -> dict:
    """Run the unit's host projection: compile with -DPIPELINK_EMIT, execute, parse what it prints.
    Units of this repo keep their device code behind #ifndef PIPELINK_EMIT and compile as plain C++ in
    a second; a unit that does not (one written for the reference's toolchain, device bodies in the
    open) is compiled as CUDA by nvcc instead."""
    source = Path(source)
    with tempfile.TemporaryDirectory() as tmp:
        exe = Path(tmp) / "emit"
        common = ["-DPIPELINK_EMIT", "-I", str(INCLUDE), *[f"-I{i}" for i in includes], *[f"-D{d}" for d in defines]]
        cmd = [os.environ.get("CXX", "g++"), "-std=c++17", "-x", "c++", "-I", str(CUDA_INCLUDE), *common, str(source), "-o", str(exe)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            arch = PROFILES[profile]["gencode"][0]           # the unit may insist on its target (a Hopper unit on sm_90a)
            cuda = [jitlink.nvcc(), "-std=c++17", "-x", "cu", "-gencode", f"arch={arch},code={arch.replace('compute', 'sm')}", "--expt-relaxed-constexpr",
                    *common, str(source), "-o", str(exe)]
            second = subprocess.run(cuda, capture_output=True, text=True)
            if second.returncode != 0:
                fail("P-COMPILE", f"{source}:emit", (proc.stderr[-1500:] + "\n--- as CUDA ---\n" + second.stderr[-1500:]))
        run = subprocess.run([str(exe)], capture_output=True, text=True)
        if run.returncode != 0:
            fail("P-ANNOTATION", str(source), run.stderr.strip() or "the manifest pass failed")
    m = json.loads(run.stdout)
    # claims in the order of their handles, those sized from a C++ type (PL_CLAIM_SMEM) behind the others and the
    # register claims last: the order the reference writes
    m["claims"].sort(key=lambda c: (2 if c.get("domain") == "regs" else int(bool(c.get("_typed"))), c.get("handle", ""), c.get("domain", "")))
    for c in m["claims"]:
        c.pop("_typed", None)
    # and endpoints: call endpoints first, then the others, each group in the order of its names
    m["endpoints"].sort(key=lambda e: ((e.get("protocol") or {}).get("kind") != "call", e.get("name", ""), e.get("direction", "")))
    if not m.get("hints"):
        m.pop("hints", None)                          # a section without entries is not written
    _check_init_warps(m, source)
    # a declaration travels with its digest (call protocols and the export records they restate)
    for rec in [ep.get("protocol") or {} for ep in m.get("endpoints", [])] + list(m["stage"].get("exports", {}).values()):
        if isinstance(rec.get("decl"), str):
            rec["decl_sha256"] = hashlib.sha256(rec["decl"].encode()).hexdigest()
    params = m["params"]
    # the layout probe: what the compiler says about the block, member by member
    probe = json.dumps([params["type"], params["bytes"], params["align"],
                        [[x["name"], x["offset"], x["bytes"]] for x in params["members"]]])
    params["sha256_of_layout_probe"] = hashlib.sha256(probe.encode()).hexdigest()
    return m


def _check_init_warps(m, source):
    """P-INIT: a barrier ring whose `init` names the physical initialising warp must name one inside its
    owner's warp claim, when that claim sits at an absolute base (docs/reference/annotations.md, pl::init)."""
    placed = {}
    for cl in m.get("claims", []):
        if cl.get("domain") == "warp" and "absolute_base" in cl:
            for role in cl.get("roles", []):
                placed[role] = (cl["absolute_base"], cl["absolute_base"] + cl["extent"]["const"])
    for i, ep in enumerate(m.get("endpoints", [])):
        init = (ep.get("protocol") or {}).get("init") or {}
        if "warp" in init and init.get("owner") in placed:
            lo, hi = placed[init["owner"]]
            if not lo <= init["warp"] < hi:
                fail("P-INIT", f"$.endpoints[{i}].protocol.init.warp",
                     f"warp {init['warp']} lies outside role {init['owner']!r}'s claim [{lo}, {hi})")


def undefined_symbols(source, profile: dict, includes=(), defines=()) -> dict:
    """External functions the unit calls and does not define, from its PTX."""
    with tempfile.TemporaryDirectory() as tmp:
        ptx = Path(tmp) / "stage.ptx"
        cmd = [jitlink.nvcc(), "-ptx", "-rdc=true", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-gencode",
               f"arch={profile['gencode'][0]},code={profile['gencode'][0]}", "-I", str(INCLUDE),
               *[f"-I{i}" for i in includes], *[f"-D{d}" for d in defines], "-o", str(ptx), str(source)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            fail("P-COMPILE", f"{source}:ptx", proc.stderr[-2000:])
        text = ptx.read_text()
    return {name: "function" for name in sorted(set(re.findall(r"^\.extern \.func[^;]*?\b(\w+)\s*(?:\(|;)", text, re.M)))}


def pack_cu(source, manifest_path=None, out=None, profile="sm_100a", includes=(), defines=(), sections=None):
    source = Path(source)
    prof = PROFILES[profile]
    includes = [str(INCLUDE), *includes]
    with tempfile.TemporaryDirectory() as tmp, ThreadPoolExecutor(3) as pool:
        obj = Path(tmp) / "stage.o"
        payload_job = pool.submit(jitlink.compile_lto, str(source), str(obj), prof, includes, defines)
        if manifest_path is None:
            undefined_job = pool.submit(undefined_symbols, source, prof, includes[1:], defines)
            manifest = emit_manifest(source, includes[1:], defines, profile)
            manifest["symbols"].update(mechanism="ptx-extern", defined_weak=[], undefined=undefined_job.result())
            manifest["payload"] = {"file": "stage.o"}
            inputs = {"tu": hashlib.sha256(source.read_bytes()).hexdigest(),
                      "annotations": hashlib.sha256((INCLUDE / "pipelink" / "stage.hpp").read_bytes()).hexdigest()}
            mechanism = "annotations"
            # sections a frontend derives in Python rather than from annotations (the tensor contracts)
            for key, value in (sections or {}).items():
                manifest[key] = json.loads(json.dumps(value))
        else:
            manifest_path = Path(manifest_path)
            manifest = json.loads(manifest_path.read_text())
            inputs = {"tu": hashlib.sha256(source.read_bytes()).hexdigest(),
                      "manifest": hashlib.sha256(manifest_path.read_bytes()).hexdigest()}
            mechanism = "declared-json"
        abi = manifest.setdefault("pipelink_abi", json.loads(json.dumps(ABI)))
        abi["target"]["profile"] = profile
        abi["target"]["lto_arch"] = prof["lto_arch"]
        schema.validate_manifest(manifest, where=manifest["stage"].get("id", str(source)))
        payload_job.result()
        payload = obj.read_bytes()
    # provenance as the reference records it (pipec/src/pipec2/schema.py:1015-1030): how the
    # manifest came to be and the digests of what it was made from
    manifest["provenance"] = {"mechanism": mechanism, "inputs": inputs}
    data = container.pack(manifest, payload)
    out = Path(out) if out else source.with_suffix(".plink")
    out.write_bytes(data)
    return out
