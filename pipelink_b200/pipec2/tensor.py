"""A stage manifest's ``tensor`` section (clause T-CONTRACT): structure, names, domains and the
placement / demand expressions.

The section is how a stage publishes a tensor for a third party's code to import (an accumulator
handed to a foreign epilogue) and what it lends that code while it runs: ``exports`` (identity
coordinates, placements as expressions over coordinates and bindings, readiness), ``imports``
(callable, demands, ``lends`` of shared memory / barriers / registers with a lifetime,
``rendezvous`` over lent barriers), ``sites`` (where the import is invoked, with the guarantees the
site gives) and ``bindings`` (link-time quantities a placement may depend on: a base column, a
slot). This module is the loading half of the reference's tensor-import planner
(pipec/src/pipec2/tensor/contracts.py, expr.py): it validates a section, evaluates its
expressions and checks an import against the export it names. Routing a connection, certifying the
program and generating the adapter is ``tensor_plan``.

Expressions are JSON lists ``[op, args...]`` over three sorts, ``int``, ``pred`` and
``bits[n]``: ``const coord bind add sub mulc divc modc eq lt le not pand por select cbits band bor
bxor shlc shrc tobits toint``. ``coord`` names a coordinate of the enclosing identity or demand
domain, ``bind`` a declared binding; the two namespaces do not mix.
"""
from __future__ import annotations

import re

SITE_GUARANTEES = ("enter_once", "single_completion", "converged", "full_warps", "no_early_return")
LEND_DOMAINS = ("smem", "barrier", "reg", "tmem", "metadata")
LEND_BINDINGS = ("relocatable", "fixed", "caller_frame")      # caller_frame: words of the caller's register frame
TENSOR_SCHEMAS = ("2.2", "3.0")
VERSION = "tensor-v2"
_BITS = re.compile(r"bits\[([1-9][0-9]*)\]\Z")

# operator -> operand kinds; "int" / "bits" / "pred" / "value" are sub-expressions, the rest literals
GRAMMAR = {
    "const": ("integer",), "cbits": ("width", "unsigned"), "coord": ("name",), "bind": ("name",),
    "add": ("int", "int"), "sub": ("int", "int"), "mulc": ("integer", "int"), "divc": ("int", "positive"),
    "modc": ("int", "positive"), "band": ("bits", "bits"), "bor": ("bits", "bits"), "bxor": ("bits", "bits"),
    "shlc": ("bits", "shift"), "shrc": ("bits", "shift"), "tobits": ("width", "int"), "toint": ("bits",),
    "select": ("pred", "value", "value"), "eq": ("int", "int"), "lt": ("int", "int"), "le": ("int", "int"),
    "not": ("pred",), "pand": ("pred", "pred"), "por": ("pred", "pred"),
}


class ExprError(ValueError):
    pass


def sort_of(expr, coords: dict, binds: dict) -> str:
    """The sort of a well-formed expression; ExprError names what is wrong with an ill-formed one.
    coords / binds: name -> sort of the coordinates and bindings in scope."""
    if not isinstance(expr, list) or not expr or expr[0] not in GRAMMAR:
        raise ExprError(f"unknown operator {expr[0] if isinstance(expr, list) and expr else expr!r}")
    op, args = expr[0], expr[1:]
    kinds = GRAMMAR[op]
    if len(args) != len(kinds):
        raise ExprError(f"{op} takes {len(kinds)} operands")
    sorts = []
    for kind, arg in zip(kinds, args):
        if kind in ("int", "bits", "pred", "value"):
            s = sort_of(arg, coords, binds)
            if (kind == "int" and s != "int") or (kind == "pred" and s != "pred") or (kind == "bits" and not _BITS.match(s)):
                raise ExprError(f"{op} wants a {kind} operand, got {s}")
            sorts.append(s)
        elif kind == "name":
            if not isinstance(arg, str):
                raise ExprError(f"{op} wants a name")
            space = coords if op == "coord" else binds
            if arg not in space:
                raise ExprError(f"{'coordinate' if op == 'coord' else 'binding'} {arg!r} is not declared here")
            sorts.append(space[arg])
        else:
            if not isinstance(arg, int) or isinstance(arg, bool) or (kind in ("positive", "width") and arg < 1) or (
                    kind in ("unsigned", "shift") and arg < 0):
                raise ExprError(f"{op} wants a {kind} literal")
            sorts.append(arg)
    if op == "const":
        return "int"
    if op in ("coord", "bind"):
        return sorts[0]
    if op in ("add", "sub", "divc", "modc", "toint"):
        return "int"
    if op == "mulc":
        return "int"
    if op in ("eq", "lt", "le", "not", "pand", "por"):
        return "pred"
    if op == "cbits":
        if args[1] >= 1 << args[0]:
            raise ExprError("cbits value does not fit its width")
        return f"bits[{args[0]}]"
    if op == "tobits":
        return f"bits[{args[0]}]"
    if op in ("band", "bor", "bxor"):
        if sorts[0] != sorts[1]:
            raise ExprError(f"{op} wants operands of one width")
        return sorts[0]
    if op in ("shlc", "shrc"):
        return sorts[0]
    if sorts[1] != sorts[2]:          # select
        raise ExprError("select wants arms of one sort")
    return sorts[1]


def evaluate(expr, env: dict):
    """Exact value of a checked expression; env: coordinate and binding names -> integers."""
    op, a = expr[0], expr[1:]
    if op == "const":
        return a[0]
    if op == "cbits":
        return a[1]
    if op in ("coord", "bind"):
        return env[a[0]]
    if op == "mulc":
        return a[0] * evaluate(a[1], env)
    if op in ("divc", "modc"):
        v = evaluate(a[0], env)
        return v // a[1] if op == "divc" else v % a[1]
    if op in ("shlc", "shrc"):
        v, width = evaluate(a[0], env), _width(a[0])
        if a[1] >= width:
            return 0
        return v >> a[1] if op == "shrc" else (v << a[1]) & ((1 << width) - 1)
    if op == "tobits":
        v = evaluate(a[1], env)
        if v < 0 or v.bit_length() > a[0]:
            raise ExprError(f"tobits operand {v} is outside [0, 2^{a[0]})")
        return v
    if op == "select":
        return evaluate(a[1], env) if evaluate(a[0], env) else evaluate(a[2], env)
    vals = [evaluate(x, env) for x in a]
    return {"add": lambda: vals[0] + vals[1], "sub": lambda: vals[0] - vals[1], "band": lambda: vals[0] & vals[1],
            "bor": lambda: vals[0] | vals[1], "bxor": lambda: vals[0] ^ vals[1], "toint": lambda: vals[0],
            "eq": lambda: int(vals[0] == vals[1]), "lt": lambda: int(vals[0] < vals[1]), "le": lambda: int(vals[0] <= vals[1]),
            "not": lambda: int(not vals[0]), "pand": lambda: int(bool(vals[0]) and bool(vals[1])),
            "por": lambda: int(bool(vals[0]) or bool(vals[1]))}[op]()


def _width(expr) -> int:
    op = expr[0]
    if op in ("cbits", "tobits"):
        return expr[1]
    if op in ("band", "bor", "bxor", "shlc", "shrc"):
        return _width(expr[1])
    if op == "select":
        return _width(expr[2])
    raise ExprError("not a bits expression")


def _domain_ok(d) -> bool:
    """A named, sorted, non-empty set of integers: a range [lo, hi) or explicit values."""
    if not isinstance(d, dict) or not isinstance(d.get("name"), str) or not (d.get("sort") == "int" or _BITS.match(str(d.get("sort")))):
        return False
    if "values" in d:
        return isinstance(d["values"], list) and len(d["values"]) > 0 and all(isinstance(v, int) for v in d["values"])
    return isinstance(d.get("lo"), int) and isinstance(d.get("hi"), int) and d["hi"] > d["lo"]


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
    if "version" in section and section["version"] != VERSION:
        bad("$.tensor.version", f"expected {VERSION!r}")

    def names_once(collection):
        seen = set()
        for i, rec in enumerate(section.get(collection, [])):
            if rec.get("name") in seen:
                bad(f"$.tensor.{collection}[{i}].name", f"duplicate {collection[:-1]} name")
            seen.add(rec.get("name"))
        return seen

    # bindings: the declared domain restates the binding's name and sort; a binding whose domain is
    # empty or of another sort is not usable by expressions
    binds = {}
    names_once("bindings")
    for i, b in enumerate(section.get("bindings", [])):
        p, dom = f"$.tensor.bindings[{i}]", b.get("domain") or {}
        usable = True
        if dom.get("name") != b.get("name"):
            bad(f"{p}.domain.name", "the domain restates the binding's name")
        if dom.get("sort") != b.get("sort"):
            bad(f"{p}.domain.sort", "the domain restates the binding's sort")
            usable = False
        elif not _domain_ok(dom):
            bad(f"{p}.domain", "a binding needs a non-empty domain")
            usable = False
        if usable and b.get("name") not in binds:
            binds[b["name"]] = b["sort"]

    def check_expr(expr, coords, path, want=None):
        try:
            s = sort_of(expr, coords, binds)
        except ExprError as err:
            bad(path, str(err))
            return
        if want == "pred" and s != "pred":
            bad(path, "expected a predicate")
        if want == "int" and s != "int":
            bad(path, "expected an integer expression")

    def coords_of(domains, path):
        coords = {}
        for j, d in enumerate(domains):
            if _domain_ok(d):
                coords[d["name"]] = d["sort"]
            else:
                bad(f"{path}[{j}]", "a coordinate needs a name, a sort and a non-empty domain")
        return coords

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

    names_once("exports")
    for i, exp in enumerate(section.get("exports", [])):
        p = f"$.tensor.exports[{i}]"
        coords = coords_of((exp.get("identity") or {}).get("coords", []), f"{p}.identity.coords")
        if not exp.get("placements"):
            bad(f"{p}.placements", "an export needs at least one placement")
        for j, pl in enumerate(exp.get("placements", [])):
            for comp, expr in sorted((pl.get("components") or {}).items()):
                check_expr(expr, coords, f"{p}.placements[{j}].components.{comp}", "int")
            if pl.get("guard") is not None:
                check_expr(pl["guard"], coords, f"{p}.placements[{j}].guard", "pred")
        declared = {b.get("name") for b in section.get("bindings", [])}
        for name in (exp.get("fixed_bindings") or {}):
            if name not in declared:
                bad(f"{p}.fixed_bindings.{name}", "not a declared binding")

    names_once("imports")
    lend_names = set()          # lends are named once per stage, across its imports
    for i, imp in enumerate(section.get("imports", [])):
        p = f"$.tensor.imports[{i}]"
        for j, s in enumerate(imp.get("sites", [])):
            if s not in site_names:
                bad(f"{p}.sites[{j}]", "unknown site")
        for j, dem in enumerate(imp.get("demands", [])):
            dp = f"{p}.demands[{j}]"
            coords = coords_of(dem.get("domain", []), f"{dp}.domain")
            for name, expr in sorted((dem.get("identity_coords") or {}).items()):
                check_expr(expr, coords, f"{dp}.identity_coords.{name}", "int")
            for field in ("participant", "position"):
                if dem.get(field) is not None:
                    check_expr(dem[field], coords, f"{dp}.{field}", "int")
            if dem.get("guard") is not None:
                check_expr(dem["guard"], coords, f"{dp}.guard", "pred")
        # a rendezvous names a barrier lend of this import; a name this import lends twice names nothing
        local, twice = {}, set()
        for j, lend in enumerate(imp.get("lends", [])):
            lp, name = f"{p}.lends[{j}]", lend.get("name")
            if name in local:
                twice.add(name)
            local.setdefault(name, lend)
            if name in lend_names:
                bad(f"{lp}.name", "duplicate lend name")
                continue
            lend_names.add(name)
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
            if lend.get("domain") == "barrier" and not lend.get("sync"):
                bad(f"{lp}.sync", "a barrier lend states its capacity and generations")
        barrier_lends = {n for n, lend in local.items() if lend.get("domain") == "barrier" and n not in twice}
        for j, r in enumerate(imp.get("rendezvous", [])):
            if r.get("barrier") not in barrier_lends:
                bad(f"{p}.rendezvous[{j}].barrier", "rendezvous requires an import barrier lend")
    return out


def check_import(export: dict, imp: dict):
    """An import against the export it is bound to: the two state the same tensor identity (result,
    version, work, dtype, interpretation, coordinates with their ranges), and every identity
    coordinate the import demands is one the export places. -> [(clause, path, message)]."""
    out = []
    ei, ii = export.get("identity") or {}, imp.get("identity") or {}
    for field in ("result", "version", "work", "dtype", "interpretation"):
        if ei.get(field) != ii.get(field):
            out.append(("T-CONTRACT", f"identity.{field}", f"export states {ei.get(field)!r}, import {ii.get(field)!r}"))
    ec = {c["name"]: (c.get("lo"), c.get("hi"), c.get("sort")) for c in ei.get("coords", [])}
    ic = {c["name"]: (c.get("lo"), c.get("hi"), c.get("sort")) for c in ii.get("coords", [])}
    if ec != ic:
        out.append(("T-CONTRACT", "identity.coords", "export and import describe different coordinate spaces"))
    for j, dem in enumerate(imp.get("demands", [])):
        for name in (dem.get("identity_coords") or {}):
            if name not in ec:
                out.append(("T-CONTRACT", f"demands[{j}].identity_coords.{name}", "the export has no such coordinate"))
        missing = sorted(set(ec) - set(dem.get("identity_coords") or {}))
        if missing:
            out.append(("T-CONTRACT", f"demands[{j}].identity_coords", f"coordinates {missing} are not addressed"))
    return out
