"""Structural validation of stage manifests (schema 3.0) and pipeline descriptions.

The vocabulary is the reference's (pipec/src/pipec2/schema.py:51-93,1205-1256): handle names
``pipelink_[A-Za-z_][A-Za-z0-9_]*``, stage IDs ``[a-z0-9]+([.-][a-z0-9]+)+``, a stage's
``symbol_prefix`` = its id lower-cased with ``.``/``-`` -> ``_`` plus ``_``, endpoint spaces
``smem|tmem|reg|gmem|none``, scopes ``cta|cluster|grid|system``, proxies ``async|generic``,
handle classes ``depth|regs|base|variant`` with owner prefixes ``channel:|reg_group:|claim:|stage:``.
"""
from __future__ import annotations

import re

from .model import ClauseFailure, PipeLinkError
from .profile import PROFILES

HANDLE_RE = re.compile(r"^pipelink_[A-Za-z_][A-Za-z0-9_]*$")
STAGE_RE = re.compile(r"^[a-z0-9]+([.-][a-z0-9]+)+$")
SPACES = {"smem", "tmem", "reg", "gmem", "none"}
SCOPES = {"cta", "cluster", "grid", "system"}
PROXIES = {"async", "generic"}
DIRECTIONS = {"produce", "consume"}
HANDLE_CLASSES = {"depth": "channel:", "regs": "reg_group:", "base": "claim:", "variant": "stage:"}
ENTRY_SIGNATURE = "void(const void* params, unsigned variant)"
SCHEMAS = ("3.0", "2.2", "2.0-draft")


def symbol_prefix(stage_id: str) -> str:
    return re.sub(r"[.-]", "_", stage_id.lower()) + "_"


class _Collector:
    def __init__(self):
        self.failures = []

    def add(self, clause, path, message, **detail):
        self.failures.append(ClauseFailure(clause, path, message, detail))

    def raise_if_any(self):
        if self.failures:
            raise PipeLinkError(self.failures)


def validate_manifest(m: dict, where: str = "manifest") -> None:
    c = _Collector()
    abi = m.get("pipelink_abi", {})
    if abi.get("schema") not in SCHEMAS:
        c.add("L-ENTRYABI", f"{where}.pipelink_abi.schema", "unsupported manifest schema")
    target = abi.get("target", {})
    if target.get("profile") not in PROFILES:
        c.add("L-LINK", f"{where}.pipelink_abi.target.profile", f"unknown profile {target.get('profile')!r}")
    st = m.get("stage", {})
    sid = st.get("id", "")
    if not STAGE_RE.match(sid):
        c.add("P-SYM", f"{where}.stage.id", f"stage id {sid!r} does not match {STAGE_RE.pattern}")
    elif st.get("symbol_prefix") != symbol_prefix(sid):
        c.add("P-SYM", f"{where}.stage.symbol_prefix", f"expected {symbol_prefix(sid)!r}")
    if st.get("entry_abi") != "v2" or st.get("entry_signature") != ENTRY_SIGNATURE:
        c.add("L-ENTRYABI", f"{where}.stage.entry_abi", "stage entries must use entry ABI v2")
    roles = st.get("roles", {})
    for name, role in roles.items():
        # an entry is any strong extern "C" symbol of the unit (the reference's own examples name theirs
        # ring_producer / ring_consumer under the prefix org_ring_producer_): uniqueness across the image
        # is what the link checks (L-SYM)
        if not role.get("entry"):
            c.add("P-SYM", f"{where}.stage.roles.{name}.entry", "a role needs an entry symbol")
        if not isinstance(role.get("warps"), int) or role["warps"] < 1:
            c.add("L-TOPO", f"{where}.stage.roles.{name}.warps", "a role needs a positive warp count")
    for i, ep in enumerate(m.get("endpoints", [])):
        p = f"{where}.endpoints[{i}]"
        if ep.get("direction") not in DIRECTIONS:
            c.add("L-PAIR", f"{p}.direction", "direction must be produce or consume")
        provided_call = (ep.get("protocol") or {}).get("kind") == "call" and ep.get("direction") == "consume"
        # an endpoint signalled or awaited inside an exported callable runs in its caller's role and names none;
        # only register tiles depend on the owning role (pipec/src/pipec2/schema.py:670-679 of the reference)
        in_callable = (ep.get("protocol") or {}).get("kind") != "call" and ep.get("space") != "reg"
        if ep.get("owner_role") not in roles and not ((provided_call or in_callable) and ep.get("owner_role") is None):
            c.add("L-OWNER", f"{p}.owner_role", f"unknown role {ep.get('owner_role')!r}")
        # a shared-completion root lists each member of its transaction sum once
        for side in ("full", "empty"):
            tx = ((ep.get("protocol") or {}).get(side) or {}).get("tx_bytes")
            if isinstance(tx, dict) and len(set(tx.get("sum", []))) != len(tx.get("sum", [])):
                c.add("L-PROTO", f"$.endpoints[{i}].protocol.{side}.tx_bytes.sum", "array entries must be unique")
        if ep.get("space") not in SPACES or ep.get("scope") not in SCOPES or ep.get("proxy") not in PROXIES:
            c.add("L-PAIR", f"{p}", "space/scope/proxy outside the vocabulary")
        for h in ep.get("binds", {}).values():
            if not HANDLE_RE.match(h):
                c.add("L-HANDLE", f"{p}.binds", f"bad handle name {h!r}")
    for i, cl in enumerate(m.get("claims", [])):
        p = f"{where}.claims[{i}]"
        if not HANDLE_RE.match(cl.get("handle", "")):
            c.add("L-HANDLE", f"{p}.handle", f"bad handle name {cl.get('handle')!r}")
        if cl.get("domain") not in PROFILES.get(target.get("profile"), {"domains": {}})["domains"]:
            c.add("L-BUDGET", f"{p}.domain", f"unknown domain {cl.get('domain')!r}")
        ext = cl.get("extent", {})
        if cl.get("domain") == "regs":
            # a register claim names the roles of one reg group and the per-thread counts it accepts
            if not cl.get("roles") or not cl.get("values") or any(not isinstance(v, int) for v in cl["values"]):
                c.add("L-REGS", f"{p}", "a regs claim needs roles and candidate values")
        elif not isinstance(ext.get("const", 0), int) or ext.get("const", 0) < 0:
            c.add("L-BUDGET", f"{p}.extent.const", "extent must be a non-negative integer")
        for r in cl.get("roles", []):
            if r not in roles:
                c.add("L-OWNER", f"{p}.roles", f"unknown role {r!r}")
    params = m.get("params", {})
    if params.get("bytes", 0) < 0 or params.get("align", 1) not in (1, 2, 4, 8, 16, 32, 64, 128):
        c.add("L-PARAMS", f"{where}.params", "bad parameter block size or alignment")
    limit = PROFILES.get(target.get("profile"), {}).get("param_limit_bytes")
    if limit is not None and params.get("bytes", 0) > limit:
        c.add("L-PARAMS", "$.params.bytes", "parameter blob exceeds the target parameter limit", limit=limit)
    # every variant row states a value for the same set of handles (the first row establishes it)
    variants = st.get("variants", [])
    for i, row in enumerate(variants[1:], start=1):
        if set(row.get("key", {})) != set(variants[0].get("key", {})):
            c.add("L-HANDLE", f"$.stage.variants[{i}].key", "variant key is incomplete")
    if "tensor" in m:
        from . import tensor
        for clause, path, message in tensor.validate_section(m["tensor"], abi.get("schema")):
            c.add(clause, path, message)
    c.raise_if_any()


def validate_pipeline(p: dict) -> None:
    c = _Collector()
    pipe = p.get("pipeline", {})
    if not pipe.get("stages"):
        c.add("L-LINK", "pipeline.stages", "a pipeline needs at least one stage")
    for name, h in pipe.get("handles", {}).items():
        if not HANDLE_RE.match(name):
            c.add("L-HANDLE", f"pipeline.handles.{name}", "bad handle name")
        cls = h.get("class")
        if cls not in HANDLE_CLASSES:
            c.add("L-HANDLE", f"pipeline.handles.{name}.class", f"unknown class {cls!r}")
        elif not str(h.get("owner", "")).startswith(HANDLE_CLASSES[cls]):
            c.add("L-HANDLE", f"pipeline.handles.{name}.owner", f"owner of a {cls} handle must start with {HANDLE_CLASSES[cls]!r}")
        if cls in ("depth", "regs") and not h.get("values"):
            c.add("L-HANDLE", f"pipeline.handles.{name}.values", f"a {cls} handle needs candidate values")
        if h.get("binding") not in ("bind", "fixed", "launch"):
            c.add("L-HANDLE", f"pipeline.handles.{name}.binding", "binding must be bind, fixed or launch")
    for name in pipe.get("forced_bindings", {}):
        if name not in pipe.get("handles", {}):
            c.add("L-HANDLE", f"pipeline.forced_bindings.{name}", "forced binding of an undeclared handle")
    for name in pipe.get("depth_priority", []):
        if pipe.get("handles", {}).get(name, {}).get("class") != "depth":
            c.add("L-HANDLE", f"pipeline.depth_priority.{name}", "not a depth handle")
    for name in pipe.get("regs_priority", []):
        if pipe.get("handles", {}).get(name, {}).get("class") != "regs":
            c.add("L-HANDLE", f"pipeline.regs_priority.{name}", "not a regs handle")
    # an exclusive entry is a pair of phase selectors: a declared phase, or `instr_*`, every phase whose name
    # starts with instr_ (two of them in one entry: every pair of different instruction phases); nothing else
    # is a pattern (the reference's rules, pipec/src/pipec2/schema.py:1285-1327)
    phases = pipe.get("phases", ["steady"])
    for i, pair in enumerate(pipe.get("exclusive", [])):
        if not isinstance(pair, list) or len(pair) != 2:
            c.add("L-PHASE", f"$.pipeline.exclusive[{i}]", "exclusive entry must contain exactly two phase selectors")
            continue
        for j, name in enumerate(pair):
            if name == "instr_*":
                if not any(ph.startswith("instr_") for ph in phases):
                    c.add("L-PHASE", f"$.pipeline.exclusive[{i}][{j}]", "instr_* matches no declared phase")
            elif isinstance(name, str) and "*" in name:
                c.add("L-PHASE", f"$.pipeline.exclusive[{i}][{j}]", "only the instr_* phase pattern is supported")
            elif name not in phases:
                c.add("L-PHASE", f"$.pipeline.exclusive[{i}][{j}]", f"unknown phase {name!r}")
        if pair[0] == pair[1] and pair[0] != "instr_*":
            c.add("L-PHASE", f"$.pipeline.exclusive[{i}]", "exclusive self-pair is invalid")
    for dom, d in pipe.get("domains", {}).items():
        if not isinstance(d.get("capacity"), int) or d["capacity"] < 0:
            c.add("L-BUDGET", f"pipeline.domains.{dom}.capacity", "a pipeline domain needs a non-negative capacity")
        if dom == "smem_page" and (not isinstance(d.get("page_bytes"), int) or d["page_bytes"] < 1):
            c.add("L-HANDLE", f"pipeline.domains.{dom}.page_bytes", "the page domain states the size of a page")
    c.raise_if_any()
