"""``pipec2 link``: packages + pipeline description -> ``pipeline.cubin`` + ``link.json``.

Phase order of the reference's driver (pipec/src/pipec2/link.py:1614-1861): load and validate ->
pair channels -> layout identity -> protocol expansion -> unify claims -> params layout -> solve
-> generate stub + dispatch -> LTO link -> receipt.
"""
from __future__ import annotations

import hashlib
import json
import tempfile
from pathlib import Path

from . import canonjson, codegen, container, contracts, jitlink, schema, tensor_plan
from .model import ClauseFailure, LinkResult, PipeLinkError
from .profile import PROFILES
from .solve import solve

INCLUDE = Path(__file__).resolve().parent / "include"      # <pipelink/...> headers of generated units

TMEM_SLOT_HANDLE = "pipelink_tmem_slot"


def _unify_claims(manifests, handles):
    """Several owners may state the same claim; the statements must agree (L-OWNER)."""
    claims, failures = {}, []
    for m in manifests:
        for cl in m.get("claims", []):
            if cl.get("domain") == "regs":
                continue                    # register claims are grouped by _reg_claims
            rec = {k: v for k, v in cl.items() if k != "roles"}
            h = cl["handle"]
            if h in claims:
                if claims[h]["rec"] != rec:
                    failures.append(ClauseFailure("L-OWNER", f"claims.{h}", "owners disagree about the claim",
                                                  {"first": claims[h]["stage"], "second": m["stage"]["id"]}))
                claims[h]["roles"] += [(m["stage"]["id"], r) for r in cl.get("roles", [])]
            else:
                claims[h] = {"rec": rec, "stage": m["stage"]["id"],
                             "roles": [(m["stage"]["id"], r) for r in cl.get("roles", [])]}
            if h not in handles:
                failures.append(ClauseFailure("L-HANDLE", f"claims.{h}", "claim handle is not declared by the pipeline"))
            elif handles[h]["class"] != "base":
                failures.append(ClauseFailure("L-HANDLE", f"claims.{h}", "a claim needs a base-class handle"))
            for dep in cl.get("extent", {}).get("per", {}):
                if handles.get(dep, {}).get("class") != "depth":
                    failures.append(ClauseFailure("L-HANDLE", f"claims.{h}.extent.per.{dep}", "extent refers to an undeclared depth handle"))
    if failures:
        raise PipeLinkError(failures)
    return claims


def _reg_claims(manifests, handles):
    """Register claims of all stages; owners that state the same group must state it identically."""
    out, failures = {}, []
    for m in manifests:
        for cl in m.get("claims", []):
            if cl.get("domain") != "regs":
                continue
            h = cl["handle"]
            if h not in handles:
                failures.append(ClauseFailure("L-HANDLE", f"claims.{h}", "claim handle is not declared by the pipeline"))
                continue
            rec = {"handle": h, "values": list(cl["values"]), "reg_group": cl.get("reg_group")}
            if h in out:
                if {k: out[h][k] for k in rec} != rec:
                    failures.append(ClauseFailure("L-OWNER", f"claims.{h}", "owners disagree about the register group"))
                out[h]["roles"] = sorted(set(out[h]["roles"]) | set(cl["roles"]))
            else:
                out[h] = dict(rec, roles=sorted(cl["roles"]))
    if failures:
        raise PipeLinkError(failures)
    return list(out.values())


def _register_audit(info: str, launch_regs):
    """What the device link reports for the linked kernel: (registers, stack bytes, spill bytes).
    The register groups were solved for a launch allocation of `launch_regs` per thread; an image
    that needs more, or that spills, does not run as solved (the reference audits the same figures
    after its link and re-solves or fails, pipec/src/pipec2/link.py:1706,1810-1825)."""
    import re
    regs = re.search(r"Used (\d+) registers", info)
    frame = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", info)
    if regs is None:
        return (-1, -1, -1)
    observed = (int(regs.group(1)), int(frame.group(1)) if frame else -1,
                int(frame.group(2)) + int(frame.group(3)) if frame else -1)
    if launch_regs is not None:
        if observed[0] > launch_regs:
            raise PipeLinkError(ClauseFailure("L-REGS", "link.register_audit",
                                              f"the linked kernel needs {observed[0]} registers per thread, the register groups were solved for {launch_regs}"))
        if observed[2] > 0:
            raise PipeLinkError(ClauseFailure("L-REGS", "link.register_audit", f"the linked kernel spills {observed[2]} bytes"))
    return observed


def _check_symbols(manifests, bindings):
    """L-SYM: no two stages define the same strong symbol, and every function a stage calls without
    defining it is either a handle the binding stub defines or another stage's strong definition
    (the reference resolves the same sets from its packages' symbol tables,
    pipec/src/pipec2/link.py:1203-1290)."""
    owners, failures = {}, []
    for m in manifests:
        for sym in m.get("symbols", {}).get("defined_strong", []):
            if sym in owners:
                failures.append(ClauseFailure("L-SYM", f'$.symbols.defined_strong["{sym}"]', "defined by two stages",
                                              {"first": owners[sym], "second": m["stage"]["id"]}))
            owners[sym] = m["stage"]["id"]
    for m in manifests:
        for sym in m.get("symbols", {}).get("undefined", {}):
            if sym in owners and owners[sym] != m["stage"]["id"]:
                continue
            if sym not in bindings:
                failures.append(ClauseFailure("L-SYM", f"{m['stage']['id']}.symbols.{sym}",
                                              "called by the stage, bound by no handle and defined by no stage"))
    if failures:
        raise PipeLinkError(failures)


def profile_scale(profile, pipe, domain):
    """Physical units per unit of a domain (an mbarrier slot is 16 bytes, a page what the pipeline states)."""
    stated = (pipe.get("domains", {}).get(domain) or {}).get("page_bytes")
    return int(stated) if stated else profile["domains"][domain].scale


def _params_layout(manifests, profile):
    """Where each stage's parameter block sits in the kernel's parameter bytes: stages in the order of
    their ids, each block on max(target alignment, its own alignment), the total rounded up to the
    largest alignment seen (the reference's rule, pipec/src/pipec2/dispatchgen.py:75-108, so the same
    packages give the same layout under either driver)."""
    base = profile["param_align"]
    entries, cursor, aggregate = [], 0, base
    for m in sorted(manifests, key=lambda m: m["stage"]["id"]):
        p = m.get("params", {"bytes": 0, "align": 1})
        align = max(p.get("align", 1), 1)
        effective = max(base, align)
        off = (cursor + effective - 1) // effective * effective
        entries.append([m["stage"]["id"], off, p.get("bytes", 0), align])
        cursor = off + p.get("bytes", 0)
        aggregate = max(aggregate, align)
    total = (cursor + aggregate - 1) // aggregate * aggregate if entries else 0
    if total > profile["param_limit_bytes"]:
        raise PipeLinkError(ClauseFailure("L-PARAMS", "params.total_bytes", f"{total} bytes exceed the {profile['param_limit_bytes']}-byte limit"))
    return {"total_bytes": total, "align": aggregate, "entries": entries}


def front_end(manifests, pipe):
    """The link phases before code generation, on documents in memory: one target profile, topology
    agreement, channel pairing, layout identity, protocol expansion, symbol resolution, claim
    unification, parameter layout and the solve. Returns what the later phases need."""
    profiles = {m["pipelink_abi"]["target"]["profile"] for m in manifests}
    if len(profiles) != 1:
        raise PipeLinkError(ClauseFailure("L-LINK", "pipelink_abi.target.profile", f"stages target different profiles: {sorted(profiles)}"))
    maths = {json.dumps(m["pipelink_abi"]["target"].get("math"), sort_keys=True) for m in manifests}
    if len(maths) != 1:
        raise PipeLinkError(ClauseFailure("L-LINK", "pipelink_abi.target.math", "one floating-point code generation mode per image"))
    profile = PROFILES[profiles.pop()]
    handles = dict(pipe.get("handles", {}))

    # the assembly: every handle an endpoint names is one the pipeline declares, before anything is paired
    # (the reference validates the same at pipec/src/pipec2/link.py:125-139, schema.validate_assembly)
    failures = []
    for m in manifests:
        for ep in m.get("endpoints", []):
            depth = (ep.get("ring") or {}).get("depth")
            if isinstance(depth, dict) and "handle" in depth and handles.get(depth["handle"], {}).get("class") != "depth":
                failures.append(ClauseFailure("L-HANDLE", f"stages.{m['stage']['id']}.endpoints.{ep['name']}.ring.depth.handle",
                                              f"ring depth handle {depth['handle']!r} is not a depth handle of the pipeline"))
        # a claim lives for the kernel, for a phase the pipeline declares, or for a tensor-event interval (a
        # record, not a string; placed like a kernel-lived claim here, which is always safe)
        for cl in m.get("claims", []):
            life = cl.get("lifetime", "kernel")
            if isinstance(life, str) and life != "kernel" and not (
                    life.startswith("phase:") and life[len("phase:"):] in pipe.get("phases", [])):
                failures.append(ClauseFailure("L-PHASE", f"stages.{m['stage']['id']}.claims.{cl.get('domain')}.{cl.get('handle')}.lifetime",
                                              f"lifetime {life!r} names no phase of the pipeline"))
    if failures:
        raise PipeLinkError(failures)
    cta_group, cluster = contracts.check_topology(manifests, profile, pipe.get("topology"))
    cluster_size = cluster[0] * cluster[1] * cluster[2]
    channels = contracts.pair_channels(manifests)
    contracts.check_compatibility(channels)
    expansions = contracts.expand_protocols(channels, manifests, cluster_size, handles)
    expansions += contracts.expand_counters(contracts.counter_channels(manifests), handles)
    for e in expansions:
        if e.get("kind") == "mbarrier" and (e.get("init") or {}).get("materializer", "dispatch") != "dispatch":
            raise PipeLinkError(ClauseFailure("L-OWNER", f"channels.{e['channel']}.protocol.init",
                                              "the generated dispatch kernel is the only barrier materializer of this build"))
        d = e.get("depth")
        if isinstance(d, dict) and "handle" in d and handles.get(d["handle"], {}).get("class") != "depth":
            raise PipeLinkError(ClauseFailure("L-HANDLE", f"channels.{e['channel']}.ring.depth", "ring depth handle is not declared"))

    # tensor connections: plan each (route, certificate, reservations) and merge what the certified
    # programs reserve into their consumers' claims, so the solve places scratch and barriers too
    tensor_records = tensor_plan.plan_pipeline(manifests, pipe)
    if tensor_records:
        manifests = [json.loads(json.dumps(m)) for m in manifests]
        for rec in tensor_records:
            consumer = next(m for m in manifests if m["stage"]["id"] == rec["consumer"])
            have = {c["handle"] for c in consumer.get("claims", [])}
            consumer.setdefault("claims", []).extend(dict(c, lifetime="kernel", roles=[]) for c in rec["claims"] if c["handle"] not in have)
    claims = _unify_claims(manifests, handles)
    uses_tmem = any(c["rec"]["domain"] == "tmem" for c in claims.values())
    if uses_tmem:  # the dispatch kernel owns the slot it publishes the allocation base through
        handles[TMEM_SLOT_HANDLE] = {"class": "base", "binding": "bind", "domain": "smem", "owner": f"claim:{TMEM_SLOT_HANDLE}"}
        claims[TMEM_SLOT_HANDLE] = {"rec": {"handle": TMEM_SLOT_HANDLE, "domain": "smem", "extent": {"const": 16, "per": {}}, "align": 16},
                                    "stage": "pipec2.dispatch", "roles": []}
    params = _params_layout(manifests, profile)
    role_warps = _role_warps(manifests, claims)
    bindings, intervals, solver = solve({h: c["rec"] for h, c in claims.items()}, handles, profile,
                                        depth_priority=pipe.get("depth_priority", []),
                                        forced=pipe.get("forced_bindings", {}),
                                        regs_priority=pipe.get("regs_priority", []),
                                        reg_claims=_reg_claims(manifests, handles), role_warps=role_warps,
                                        pipeline_domains=pipe.get("domains", {}), exclusive=[tuple(e) for e in pipe.get("exclusive", [])])
    # a named-barrier hand-off: both ends' storage claims must have been solved to the same bytes
    for name, ((ps, pe), (cs, ce)) in channels.items():
        if (pe.get("protocol") or {}).get("kind") != "named_barrier":
            continue
        places = []
        for ep in (pe, ce):
            h = (ep.get("binds") or {}).get("base")
            if h in bindings and h in claims:
                places.append(bindings[h][0] * profile_scale(profile, pipe, claims[h]["rec"]["domain"]))
        if len(places) == 2 and places[0] != places[1]:
            raise PipeLinkError(ClauseFailure("L8", f"channels.{name}.endpoint.physical_identity",
                                              "the two ends of the hand-off hold different storage", {"bytes": places}))
    for rec in tensor_records:       # a lend no certified program touches claims nothing: its handle resolves to 0
        for h in rec["unused_handles"]:
            bindings.setdefault(h, [0, "unused"])
    generated_symbols = {e["trampoline"]["caller"]: None for e in expansions if "trampoline" in e}
    for rec in tensor_records:
        generated_symbols.update({rec["callable"] + suffix: None for suffix in ("", "_ready", "_done")})
    _check_symbols(manifests, {**bindings, **generated_symbols})
    return {"tensor": tensor_records, "profile": profile, "handles": handles, "cta_group": cta_group, "cluster": cluster, "expansions": expansions,
            "claims": claims, "uses_tmem": uses_tmem, "params": params, "role_warps": role_warps, "bindings": bindings,
            "intervals": intervals, "solver": solver}


def _role_warps(manifests, claims):
    """role -> (warp claim handle, warps, offset inside the claim). A warp claim may cover several
    roles of its stage; they occupy it in the order the claim lists them."""
    out = {}
    for h, c in claims.items():
        if c["rec"]["domain"] != "warp":
            continue
        offset = 0
        for stage_id, rname in c["roles"]:
            m = next(m for m in manifests if m["stage"]["id"] == stage_id)
            warps = m["stage"]["roles"][rname]["warps"]
            out[rname] = (h, warps, offset)
            offset += warps
        if c["roles"] and offset != c["rec"]["extent"]["const"]:
            raise PipeLinkError(ClauseFailure("L-TOPO", f"claims.{h}", "warp claim extent differs from its roles' warp counts"))
    return out


def link(pipeline_path, out_dir, *, device_link=True):
    pipeline_path, out_dir = Path(pipeline_path), Path(out_dir)
    spec = json.loads(pipeline_path.read_text())
    schema.validate_pipeline(spec)
    pipe = spec["pipeline"]
    manifests, payloads, input_hashes = [], [], {}
    for st in pipe["stages"]:
        path = (pipeline_path.parent / st["artifact_path"]).resolve()
        m, payload = container.read(path)
        schema.validate_manifest(m, where=m["stage"].get("id", str(path)))
        if m["stage"]["id"] != st["stage_id"]:
            raise PipeLinkError(ClauseFailure("L-LINK", f"pipeline.stages.{st['stage_id']}", f"package holds stage {m['stage']['id']!r}"))
        manifests.append(m)
        payloads.append(payload)
        input_hashes[st["stage_id"]] = hashlib.sha256(path.read_bytes()).hexdigest()
    fe = front_end(manifests, pipe)
    profile, handles, cta_group, cluster, expansions = fe["profile"], fe["handles"], fe["cta_group"], fe["cluster"], fe["expansions"]
    claims, uses_tmem, params, bindings, intervals, solver = (fe["claims"], fe["uses_tmem"], fe["params"], fe["bindings"],
                                                              fe["intervals"], fe["solver"])

    # roles: warp interval from the role's warp claim, params offset from the layout
    offsets = {e[0]: e[1] for e in params["entries"]}
    # a role without a warp claim takes the next warps behind the claimed ones, in declaration order
    # (the smallest images, one role and nothing to solve, carry no claim at all)
    roles, covered, unplaced = [], 0, []
    for m in manifests:
        for rname, r in m["stage"]["roles"].items():
            rec = {"stage": m["stage"]["id"], "role": rname, "entry": r["entry"], "warps": r["warps"],
                   "params_offset": offsets[m["stage"]["id"]], "variant": 0}
            if rname in fe["role_warps"]:
                handle, warps, inside = fe["role_warps"][rname]
                rec["warp_lo"] = bindings[handle][0] + inside
                roles.append(rec)
            else:
                unplaced.append(rec)
            covered += r["warps"]
    next_warp = max((r["warp_lo"] + r["warps"] for r in roles), default=0)
    for rec in unplaced:
        rec["warp_lo"], next_warp = next_warp, next_warp + rec["warps"]
        roles.append(rec)
    for rec in roles:
        rec["warp_hi"] = rec["warp_lo"] + rec.pop("warps")
    if not roles:
        raise PipeLinkError(ClauseFailure("L-TOPO", "pipeline.stages", "an image needs at least one role"))
    roles.sort(key=lambda r: r["warp_lo"])
    threads = 32 * covered
    tmem_cols = 0
    if uses_tmem:
        hw = max(iv["hi"] for iv in intervals["tmem"])
        tmem_cols = 32
        while tmem_cols < hw:
            tmem_cols *= 2
    smem_hw = solver["high_water"].get("smem", 0)
    generated = {
        "binding_stub.cu": codegen.binding_stub(bindings, [e["trampoline"] for e in expansions if "trampoline" in e]),
        "dispatch.cu": codegen.dispatch(threads=threads, params_total=params["total_bytes"], params_align=params["align"], roles=roles,
                                        expansions=expansions, bindings=bindings, tmem_columns=tmem_cols,
                                        tmem_slot=bindings.get(TMEM_SLOT_HANDLE, [0])[0], tmem_warp=roles[0]["warp_lo"],
                                        cta_group=cta_group, cluster=cluster, reg_groups=solver.get("reg_groups", []),
                                        launch_regs=solver.get("launch_regs"),
                                        extra_barriers={h: c["rec"]["init_count"] for h, c in claims.items()
                                                        if c["rec"]["domain"] == "mbarrier" and "init_count" in c["rec"]}),
    }
    if fe["tensor"]:
        by_role = {r["role"]: (r["warp_lo"], r["warp_hi"] - r["warp_lo"]) for r in roles}
        generated["tensor_adapters.cu"] = tensor_plan.adapters_unit(fe["tensor"], by_role)
    out_dir.mkdir(parents=True, exist_ok=True)
    gen_dir = out_dir / "generated"
    gen_dir.mkdir(exist_ok=True)
    for name, text in generated.items():
        (gen_dir / name).write_text(text)
    observed = (-1, -1, -1)
    if device_link:
        objects = [(m["stage"]["id"], p) for m, p in zip(manifests, payloads)]
        with tempfile.TemporaryDirectory() as tmp:
            for name in generated:
                obj = Path(tmp) / (name + ".o")
                jitlink.compile_lto(str(gen_dir / name), str(obj), profile, [INCLUDE])
                objects.append((name, obj.read_bytes()))
        cubin, info = jitlink.link(objects, profile["sm"], extra=["-Xptxas=-v"])
        (out_dir / "pipeline.cubin").write_bytes(cubin)
        (out_dir / "nvjitlink.log").write_text(info)
        observed = _register_audit(info, solver.get("launch_regs"))
    result = LinkResult(
        kernel_symbol="pipelink_kernel", threads=threads,
        regs_cap=solver.get("launch_regs") or min(255, 65536 // max(threads, 1) // 8 * 8),
        dyn_smem_bytes=smem_hw, cluster=tuple(cluster), params=params, bindings=bindings, variants={},
        intervals=intervals, protocol_expansions=expansions, observed=observed, input_hashes=input_hashes,
        generated_hashes={k: hashlib.sha256(v.encode()).hexdigest() for k, v in generated.items()},
        solver=solver, roles=roles, tmem_columns=tmem_cols, tensor=fe["tensor"] or None)
    (out_dir / "link.json").write_text(canonjson.dumps(result.to_json_obj()))
    return result
