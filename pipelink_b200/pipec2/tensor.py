"""Structural checks of a stage manifest's ``tensor`` section (clause T-CONTRACT).

The section is how a stage publishes a tensor for a third party's code to import (an accumulator
handed to a foreign epilogue) and what it lends that code while it runs: ``exports`` (identity,
placements, readiness), ``imports`` (callable, demands, ``lends`` of shared memory / barriers /
registers with a lifetime, ``rendezvous`` over lent barriers), ``sites`` (where the import is
invoked, with the guarantees the site gives) and ``bindings``. This module validates the
section's own consistency, the part of the reference's contract loader
(pipec/src/pipec2/tensor/contracts.py) that its negative fixtures 16-19 exercise; planning
adapters between placements is not part of this build.
"""
from __future__ import annotations

SITE_GUARANTEES = ("enter_once", "converged", "full_warps", "no_early_return")
LEND_DOMAINS = ("smem", "barrier", "reg", "tmem")
LEND_BINDINGS = ("relocatable", "fixed")
TENSOR_SCHEMAS = ("2.2", "3.0")


def validate_section(section, schema_version):
    """-> [(clause, path, message)]; empty when the section is well formed."""
    out = []

    def bad(path, message):
        out.append(("T-CONTRACT", path, message))

    if schema_version not in TENSOR_SCHEMAS:
        bad("$.tensor", "tensor contracts require schema 2.2 or 3.0")
        return out
    if not isinstance(section, dict):
        bad("$.tensor", "expected an object")
        return out
    site_names = set()
    for i, site in enumerate(section.get("sites", [])):
        p = f"$.tensor.sites[{i}]"
        if site.get("name") in site_names:
            bad(f"{p}.name", "duplicate site name")
        site_names.add(site.get("name"))
        seen = set()
        for j, g in enumerate(site.get("guarantees", [])):
            if g not in SITE_GUARANTEES:
                bad(f"{p}.guarantees[{j}]", "unexpected value")
            elif g in seen:
                bad(f"{p}.guarantees[{j}]", "duplicate guarantee")
            seen.add(g)
    export_names = set()
    for i, exp in enumerate(section.get("exports", [])):
        p = f"$.tensor.exports[{i}]"
        if exp.get("name") in export_names:
            bad(f"{p}.name", "duplicate export name")
        export_names.add(exp.get("name"))
        coords = [c.get("name") for c in (exp.get("identity") or {}).get("coords", [])]
        if len(set(coords)) != len(coords):
            bad(f"{p}.identity.coords", "duplicate coordinate name")
        if not exp.get("placements"):
            bad(f"{p}.placements", "an export needs at least one placement")
    for i, imp in enumerate(section.get("imports", [])):
        p = f"$.tensor.imports[{i}]"
        for j, s in enumerate(imp.get("sites", [])):
            if s not in site_names:
                bad(f"{p}.sites[{j}]", "unknown site")
        lends, barrier_lends = {}, set()
        for j, lend in enumerate(imp.get("lends", [])):
            lp = f"{p}.lends[{j}]"
            name = lend.get("name")
            if name in lends:
                bad(f"{lp}.name", "duplicate lend name")
                lends[name] = None          # neither of the two can be referred to any more
                barrier_lends.discard(name)
                continue
            lends[name] = lend
            if lend.get("domain") not in LEND_DOMAINS:
                bad(f"{lp}.domain", "unexpected value")
            if lend.get("binding") not in LEND_BINDINGS:
                bad(f"{lp}.binding", "unexpected value")
            loc = lend.get("location") or {}
            if lend.get("binding") == "relocatable" and not loc.get("handle"):
                bad(f"{lp}.location.handle", "relocatable lend requires a handle")
            if lend.get("binding") == "fixed" and loc.get("base") is None and not loc.get("handle"):
                bad(f"{lp}.location", "fixed lend requires a base or a named location")
            if not isinstance(lend.get("extent"), int) or lend["extent"] < 1:
                bad(f"{lp}.extent", "a lend needs a positive extent")
            if lend.get("domain") == "barrier":
                barrier_lends.add(name)
                if not lend.get("sync"):
                    bad(f"{lp}.sync", "a barrier lend states its capacity and generations")
        for j, r in enumerate(imp.get("rendezvous", [])):
            if r.get("barrier") not in barrier_lends:
                bad(f"{p}.rendezvous[{j}].barrier", "rendezvous requires an import barrier lend")
    return out
