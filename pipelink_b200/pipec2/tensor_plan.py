"""The planning half of tensor imports: route, certify and lower the adapter between an exported
tensor's placement and an import's demand.

A producer exports a logical tensor (identity coordinates) with a placement: tensor memory
(``lane`` / ``column`` of 32-bit cells relative to the source address), immutable shared memory
(``byte`` offset from the source pointer) or a register frame (``participant`` / ``position``). A
consumer demands positions: participant ``t`` holds, at private position ``p``, the element whose
identity coordinates the demand states as expressions of ``(t, p)``. For one connection the planner
tries a fixed structural order of routes, each a short program over typed primitives:

    direct_receipt      tmem   every participant already sits on the lane that holds its elements,
                               in position order: tcgen05.ld straight into the destination
    shared_direct       smem   shared -> register loads at the composed address
    frame_local         regs   the producer's frame of the same participant, re-indexed
    staged_constructed  tmem   receipt of the own lane, store to lent scratch through an XOR shear
                               chosen by exact per-warp bank-conflict scoring, rendezvous, load

Every proposal is replayed by ``certify`` on a finite machine model built from the export's
placement (every participant, every position): the terminal demand must hold, no scratch word is
written twice, and what the C lowering of every expression computes equals the expression's exact
value at every point. The program's expressions are the ones ``lower`` prints, so the certificate
is about the code that is generated. Resources are what the certified program touched (scratch
high-water mark, barrier generations), held against the import's lends.

The reference plans the same connections with a larger vocabulary (cross-lane shuffles, bounded
solver search, memory views) and lowers through a third-party tile compiler
(pipec/src/pipec2/tensor/plan.py, routes.py, machine.py, check.py, lower.py;
docs/reference/tensor-imports.md "Planning"); here the routes above are built constructively and
lowered to CUDA text directly. Outcome names and clauses are the reference's: ``MODEL_SAT``,
``CONTRACT_INVALID`` (T-CONTRACT), ``UNSUPPORTED_MODEL`` (T-MODEL), ``RESOURCE_ENVELOPE`` (T-PLAN),
``T-PLAN-RENDEZVOUS``, ``T-PLAN-FRAME``.
"""
from __future__ import annotations

import hashlib
import itertools
import json

from . import tensor
from .model import ClauseFailure, PipeLinkError

ROUTE_ORDER = ("direct_receipt", "shared_direct", "frame_local", "staged_constructed")
WORD_DTYPES = ("f32", "i32", "u32")
C_TYPES = {"f32": "float", "i32": "int", "u32": "unsigned"}
RECEIPT_CHUNKS = (32, 16, 8, 4, 2, 1)


class Infeasible(Exception):
    """A route does not apply; `outcome` is the reference's outcome name, `facts` what is missing."""

    def __init__(self, outcome, reason, clause="T-PLAN", facts=None):
        super().__init__(reason)
        self.outcome, self.reason, self.clause, self.facts = outcome, reason, clause, facts or {}


# ---------------------------------------------------------------- expressions
def substitute(expr, mapping):
    """The expression with every ["coord", name] of `mapping` replaced by mapping[name]."""
    if not isinstance(expr, list):
        return expr
    if expr[0] == "coord" and expr[1] in mapping:
        return mapping[expr[1]]
    return [expr[0]] + [substitute(a, mapping) if isinstance(a, list) else a for a in expr[1:]]


def bind_values(expr, values):
    """The expression with every ["bind", name] replaced by its fixed value."""
    if not isinstance(expr, list):
        return expr
    if expr[0] == "bind":
        if expr[1] not in values:
            raise Infeasible("UNSUPPORTED_MODEL", f"binding {expr[1]!r} is a runtime input", "T-MODEL")
        return ["const", values[expr[1]]]
    return [expr[0]] + [bind_values(a, values) if isinstance(a, list) else a for a in expr[1:]]


def expr_to_c(expr, names):
    """C text of an expression over int variables `names` (coordinate -> C identifier)."""
    op, a = expr[0], expr[1:]
    c = lambda e: expr_to_c(e, names)
    if op == "const":
        return f"({a[0]})" if a[0] < 0 else str(a[0])
    if op == "cbits":
        return f"{a[1]}u"
    if op == "coord":
        return names[a[0]]
    if op == "mulc":
        return f"({a[0]} * {c(a[1])})"
    if op in ("divc", "modc"):
        return f"({c(a[0])} {'/' if op == 'divc' else '%'} {a[1]})"
    if op in ("add", "sub"):
        return f"({c(a[0])} {'+' if op == 'add' else '-'} {c(a[1])})"
    if op in ("band", "bor", "bxor"):
        return f"({c(a[0])} {dict(band='&', bor='|', bxor='^')[op]} {c(a[1])})"
    if op == "shlc":
        return f"(({c(a[0])} << {a[1]}) & {(1 << tensor._width(a[0])) - 1}u)"
    if op == "shrc":
        return f"({c(a[0])} >> {a[1]})"
    if op == "tobits":
        return f"((unsigned)({c(a[1])}))"
    if op == "toint":
        return f"((int)({c(a[0])}))"
    if op == "select":
        return f"({c(a[0])} ? {c(a[1])} : {c(a[2])})"
    if op in ("eq", "lt", "le"):
        return f"({c(a[0])} {dict(eq='==', lt='<', le='<=')[op]} {c(a[1])})"
    if op == "not":
        return f"(!{c(a[0])})"
    if op in ("pand", "por"):
        return f"({c(a[0])} {'&&' if op == 'pand' else '||'} {c(a[1])})"
    raise Infeasible("UNSUPPORTED_MODEL", f"operator {op!r} has no C lowering", "T-LOWER")


def c_value(expr, env):
    """What the C text of `expr_to_c` computes (truncating division, 32-bit unsigned bit ops):
    compared with `tensor.evaluate` at every point a program touches."""
    op, a = expr[0], expr[1:]
    if op in ("divc", "modc"):
        v = c_value(a[0], env)
        q = abs(v) // a[1] * (1 if v >= 0 else -1)
        return q if op == "divc" else v - q * a[1]
    if op == "tobits":
        return c_value(a[1], env) & 0xFFFFFFFF
    if op in ("const", "cbits", "coord", "bind"):
        return tensor.evaluate(expr, env)
    if op == "mulc":
        return a[0] * c_value(a[1], env)
    if op == "shlc":
        return (c_value(a[0], env) << a[1]) & ((1 << tensor._width(a[0])) - 1)
    if op == "shrc":
        return c_value(a[0], env) >> a[1]
    if op == "select":
        return c_value(a[1], env) if c_value(a[0], env) else c_value(a[2], env)
    v = [c_value(x, env) for x in a]
    return {"add": lambda: v[0] + v[1], "sub": lambda: v[0] - v[1], "band": lambda: v[0] & v[1], "bor": lambda: v[0] | v[1],
            "bxor": lambda: v[0] ^ v[1], "toint": lambda: v[0], "eq": lambda: int(v[0] == v[1]), "lt": lambda: int(v[0] < v[1]),
            "le": lambda: int(v[0] <= v[1]), "not": lambda: int(not v[0]), "pand": lambda: int(bool(v[0]) and bool(v[1])),
            "por": lambda: int(bool(v[0]) or bool(v[1]))}[op]()


def _value(expr, env):
    """Exact value, and the proof obligation that the C text computes the same."""
    exact = tensor.evaluate(expr, env)
    if c_value(expr, env) != exact:
        raise Infeasible("LOWERING_UNSUPPORTED", f"C arithmetic differs from the exact value at {env}", "T-LOWER")
    return exact


def _range(d):
    return list(d["values"]) if "values" in d else list(range(d["lo"], d["hi"]))


# ---------------------------------------------------------------- the connection, normalised
class Connection:
    """An export's placement and an import's demand over one finite space."""

    # component names of the reference's units ("dp/column", "byte" addresses) beside this build's own
    ALIASES = {"dp": "lane", "address": "byte"}

    def __init__(self, export, imp, site, bindings=None, runtime=None):
        """bindings: {name: value} known at link time. runtime: {name: {"values": [...], "units": ...}}, bindings
        whose value the producer publishes at run time; one whose unit is `column` is what the tensor-memory
        source handle carries, so the placement's columns are planned relative to it (checked in every world)."""
        self.export, self.imp, self.site = export, imp, site
        failures = tensor.check_import(export, imp)
        if failures:
            raise Infeasible("CONTRACT_INVALID", "; ".join(f"{p}: {m}" for _c, p, m in failures), "T-CONTRACT")
        ident = export["identity"]
        if ident.get("dtype") not in WORD_DTYPES:
            raise Infeasible("UNSUPPORTED_MODEL", f"element type {ident.get('dtype')!r}: this build moves 32-bit words", "T-MODEL")
        self.dtype = ident["dtype"]
        self.coords = ident["coords"]
        if len(export.get("placements", [])) != 1 or len(imp.get("demands", [])) != 1:
            raise Infeasible("UNSUPPORTED_MODEL", "one placement and one demand per connection", "T-MODEL")
        fixed = dict(bindings or {})
        fixed.update(export.get("fixed_bindings") or {})
        self.placement = export["placements"][0]
        self.space = self.placement.get("space")
        runtime = {k: v for k, v in (runtime or {}).items() if k not in fixed}
        worlds = [dict(zip(runtime, vs)) for vs in itertools.product(*[r["values"] for r in runtime.values()])] or [{}]
        if len(worlds) > 64:
            raise Infeasible("UNSUPPORTED_MODEL", f"{len(worlds)} binding worlds", "T-MODEL")

        def bias(world):
            return sum(v for k, v in world.items() if runtime[k].get("units") == "column")

        def in_world(world):
            return {self.ALIASES.get(k, k): bind_values(e, {**fixed, **world}) for k, e in self.placement["components"].items()}

        self.components = in_world(worlds[0])
        if bias(worlds[0]) and "column" in self.components:
            self.components["column"] = ["add", self.components["column"], ["const", -bias(worlds[0])]]
        if len(worlds) > 1:
            names = [c["name"] for c in ident["coords"]]
            for world in worlds[1:]:
                other = in_world(world)
                for point in itertools.product(*[_range(c) for c in ident["coords"]]):
                    e = dict(zip(names, point))
                    for k, expr in other.items():
                        shift = bias(world) if k == "column" else 0
                        if tensor.evaluate(expr, e) - shift != tensor.evaluate(self.components[k], e):
                            raise Infeasible("UNSUPPORTED_MODEL", f"placement component {k} depends on a run-time binding other than as the source's base column", "T-MODEL")
        self.guard = bind_values(self.placement["guard"], fixed) if self.placement.get("guard") is not None else None
        dem = imp["demands"][0]
        if dem.get("guard") is not None:
            raise Infeasible("UNSUPPORTED_MODEL", "guarded demands", "T-MODEL")
        dom = list(dem.get("domain", []))
        if len(dom) == 1:          # one element per participant: the position is the single point 0
            dom.append({"name": "pl_position", "lo": 0, "hi": 1, "sort": "int"})
        if len(dom) != 2:
            raise Infeasible("UNSUPPORTED_MODEL", "a positions demand ranges over (participant, position)", "T-MODEL")
        self.t, self.p = dom[0], dom[1]
        self.participants, self.positions = _range(self.t), _range(self.p)
        if self.participants != list(range(len(self.participants))) or self.positions != list(range(len(self.positions))):
            raise Infeasible("UNSUPPORTED_MODEL", "participants and positions count from 0", "T-MODEL")
        # the demand's two coordinates ARE the participant and the private position
        for field, coord in (("participant", self.t), ("position", self.p)):
            e = dem.get(field) or ["coord", coord["name"]]
            for t, p in ((0, 0), (self.participants[-1], self.positions[-1]), (self.participants[-1] // 2, 1 % len(self.positions))):
                if tensor.evaluate(e, {self.t["name"]: t, self.p["name"]: p}) != (t if field == "participant" else p):
                    raise Infeasible("UNSUPPORTED_MODEL", f"demand {field} is not the demand's own coordinate", "T-MODEL")
        self.identity_of = {k: bind_values(e, fixed) for k, e in dem["identity_coords"].items()}
        threads = site.get("participants")
        if threads is not None and threads != len(self.participants):
            raise Infeasible("CONTRACT_INVALID", f"the site has {threads} participants, the demand {len(self.participants)}", "T-CONTRACT")
        self.lends = {lend["name"]: lend for lend in imp.get("lends", [])}

    # identity and source location of what (t, p) demands
    def env(self, t, p):
        return {self.t["name"]: t, self.p["name"]: p}

    def composed(self, component):
        """The export's placement component as an expression of the demand's (t, p)."""
        return substitute(self.components[component], self.identity_of)

    def identity(self, t, p):
        e = self.env(t, p)
        return tuple(_value(self.identity_of[c["name"]], e) for c in self.coords)

    def placed(self):
        """{source location: identity} of the export over its whole identity domain."""
        names = [c["name"] for c in self.coords]
        comps = sorted(self.components)
        out = {}
        for point in itertools.product(*[_range(c) for c in self.coords]):
            e = dict(zip(names, point))
            if self.guard is not None and not tensor.evaluate(self.guard, e):
                continue
            loc = tuple(tensor.evaluate(self.components[k], e) for k in comps)
            if loc in out:
                raise Infeasible("CONTRACT_INVALID", f"placement puts {out[loc]} and {point} at {dict(zip(comps, loc))}", "T-CONTRACT")
            out[loc] = point
        return comps, out

    def lend(self, domain, purpose=None):
        for lend in self.lends.values():
            if lend.get("domain") == domain and (purpose is None or lend.get("purpose") == purpose):
                return lend
        return None


# ---------------------------------------------------------------- routes
def _t(conn):
    return ["coord", conn.t["name"]]


def _p(conn):
    return ["coord", conn.p["name"]]


def _receipt_lane_checks(conn):
    if conn.space != "tmem":
        raise Infeasible("NOT_APPLICABLE", "not a tensor-memory export")
    if len(conn.participants) != 128:
        raise Infeasible("RESOURCE_ENVELOPE", "a tensor-memory receipt is four warps on 128 lanes", facts={"participants": 128})
    if not conn.site.get("warpgroup_aligned"):
        raise Infeasible("RESOURCE_ENVELOPE", "warp w reads lanes 32 (w mod 4)..: the site's role must start on a multiple of four warps",
                         facts={"role_warp_align": 4})


def route_direct_receipt(conn):
    _receipt_lane_checks(conn)
    lane, col = conn.composed("lane"), conn.composed("column")
    P = len(conn.positions)
    c0 = tensor.evaluate(col, conn.env(0, 0))
    for t in conn.participants:
        for p in conn.positions:
            e = conn.env(t, p)
            if tensor.evaluate(lane, e) != t or tensor.evaluate(col, e) != c0 + p:
                raise Infeasible("BOUNDED_UNSAT", f"participant {t} position {p} is not cell (lane {t}, column {c0 + p})")
    return [{"op": "tmem_receipt", "lane": _t(conn), "column": ["add", ["const", c0], ["coord", "i"]], "count": P, "to": "dest"}]


def route_shared_direct(conn):
    if conn.space != "smem":
        raise Infeasible("NOT_APPLICABLE", "not a shared-memory export")
    return [{"op": "smem_load", "space": "source", "byte": conn.composed("byte"), "count": len(conn.positions), "to": "dest"}]


def route_frame_local(conn):
    if conn.space != "regs":
        raise Infeasible("NOT_APPLICABLE", "not a register export")
    frame = conn.lend("reg", "frame")
    comps, placed = conn.placed()
    words = 1 + max(loc[comps.index("position")] for loc in placed)
    if frame is None or frame["extent"] < words:
        raise Infeasible("RESOURCE_ENVELOPE", "a register export needs one frame lend with enough positions per participant",
                         "T-PLAN-FRAME", {"frame_words": words})
    who, where = conn.composed("participant"), conn.composed("position")
    for t in conn.participants:
        for p in conn.positions:
            if tensor.evaluate(who, conn.env(t, p)) != t:
                raise Infeasible("BOUNDED_UNSAT", f"participant {t} position {p} lives in another participant's frame")
    return [{"op": "frame_load", "index": where, "count": len(conn.positions), "to": "dest"}]


def _shear(width_bits, modulus, t_expr):
    return ["tobits", width_bits, ["modc", t_expr, modulus]]


def _bank_score(words_per_instruction):
    """Sum over warp-wide instructions of the worst bank's multiplicity (1 = conflict free)."""
    total = 0
    for words in words_per_instruction:
        banks = {}
        for w in set(words):          # lanes reading one word are served by one broadcast
            banks[w % 32] = banks.get(w % 32, 0) + 1
        total += max(banks.values())
    return total


def route_staged_constructed(conn):
    _receipt_lane_checks(conn)
    scratch, barrier = conn.lend("smem"), conn.lend("barrier")
    comps, placed = conn.placed()
    li, ci = comps.index("lane"), comps.index("column")
    cols = sorted({loc[ci] for loc in placed})
    c_lo, C = cols[0], cols[-1] - cols[0] + 1
    if max(loc[li] for loc in placed) >= 128:
        raise Infeasible("UNSUPPORTED_MODEL", "lanes above 127", "T-MODEL")
    if scratch is None or barrier is None:
        raise Infeasible("RESOURCE_ENVELOPE", "staging needs a shared-memory lend and a barrier lend",
                         facts={"smem_bytes": 128 * C * 4, "barrier_generations": 3})
    lane2, col2 = conn.composed("lane"), ["sub", conn.composed("column"), ["const", c_lo]]
    t, i = _t(conn), ["coord", "i"]
    pow2 = C & (C - 1) == 0
    bits = max(C.bit_length() - 1, 1)
    family = [0] + ([min(C, 32)] if pow2 and C > 1 else [])
    best = None
    for modulus in family:
        if modulus:
            word = lambda lane, col: ["add", ["mulc", C, lane], ["toint", ["bxor", ["tobits", bits, col], _shear(bits, modulus, lane)]]]
        else:
            word = lambda lane, col: ["add", ["mulc", C, lane], col]
        store, load = word(t, i), word(lane2, col2)
        score = 0
        for w0 in range(0, 128, 32):
            score += _bank_score([[tensor.evaluate(store, {conn.t["name"]: w0 + l, "i": k}) for l in range(32)] for k in range(C)])
            score += _bank_score([[tensor.evaluate(load, conn.env(w0 + l, p)) for l in range(32)] for p in conn.positions])
        if best is None or score < best[0]:
            best = (score, modulus, store, load)
    score, modulus, store, load = best
    return [{"op": "tmem_receipt", "lane": t, "column": ["add", ["const", c_lo], i], "count": C, "to": "r"},
            {"op": "smem_store", "space": "scratch", "word": store, "count": C, "from": "r"},
            {"op": "rendezvous", "barrier": barrier["name"]},
            {"op": "smem_load", "space": "scratch", "word": load, "count": len(conn.positions), "to": "dest",
             "shear_modulus": modulus, "bank_score": score, "conflict_free_score": 4 * (C + len(conn.positions))}]


ROUTES = {"direct_receipt": route_direct_receipt, "shared_direct": route_shared_direct, "frame_local": route_frame_local,
          "staged_constructed": route_staged_constructed}


# ---------------------------------------------------------------- the checker
def certify(program, conn):
    """Replay on the finite machine: -> {"scratch_bytes", "barrier_generations"} of what the
    program touched. Raises Infeasible (CHECK_FAILED) with the first participant / position at
    which the terminal demand does not hold."""
    comps, placed = conn.placed()
    tn = conn.t["name"]
    regs = {t: {} for t in conn.participants}
    dest = {t: {} for t in conn.participants}
    scratch, high_water, generations = {}, 0, 0

    def fail(msg):
        raise Infeasible("CHECK_FAILED", msg, "T-PLAN")

    for step in program:
        op = step["op"]
        if op == "tmem_receipt":
            for t in conn.participants:
                lane = _value(step["lane"], {tn: t})
                if lane != t or not conn.site.get("warpgroup_aligned"):
                    fail(f"participant {t} cannot read lane {lane}")
                for k in range(step["count"]):
                    loc = {"lane": lane, "column": _value(step["column"], {tn: t, "i": k})}
                    (dest if step["to"] == "dest" else regs)[t][k] = placed.get(tuple(loc[c] for c in comps))
        elif op == "smem_store":
            for t in conn.participants:
                for k in range(step["count"]):
                    w = _value(step["word"], {tn: t, "i": k})
                    if w < 0 or w in scratch:
                        fail(f"scratch word {w} written twice (participant {t}, element {k})")
                    scratch[w] = regs[t].get(k)
                    high_water = max(high_water, 4 * (w + 1))
        elif op == "rendezvous":
            generations += 1
        elif op == "smem_load":
            for t in conn.participants:
                for p in range(step["count"]):
                    if step["space"] == "scratch":
                        if generations == 0:
                            fail("scratch is read before the rendezvous that publishes it")
                        dest[t][p] = scratch.get(_value(step["word"], conn.env(t, p)))
                    else:
                        dest[t][p] = placed.get((_value(step["byte"], conn.env(t, p)),))
        elif op == "frame_load":
            for t in conn.participants:
                for p in range(step["count"]):
                    loc = {"participant": t, "position": _value(step["index"], conn.env(t, p))}
                    dest[t][p] = placed.get(tuple(loc[c] for c in comps))
        else:
            fail(f"unknown primitive {op!r}")
    for t in conn.participants:
        for p in conn.positions:
            want = conn.identity(t, p)
            if dest[t].get(p) != want:
                fail(f"participant {t} position {p} holds {dest[t].get(p)}, the demand is {want}")
    return {"scratch_bytes": high_water, "barrier_generations": generations}


# ---------------------------------------------------------------- planning one connection
def _rendezvous_events(conn):
    events = [r.get("event") for r in conn.imp.get("rendezvous", [])]
    # the two outer events: by this build's names, or as the contracts name them (the export's readiness
    # event and the import's completion event, as the reference's units do)
    wanted = ("ready", "done")
    readiness = conn.export.get("readiness")
    named = (readiness.get("after") if isinstance(readiness, dict) else None, conn.imp.get("completion"))
    if all(named) and all(e in events for e in named):
        wanted = named
    missing = [e for e in wanted if e not in events]
    if missing:
        raise PipeLinkError(ClauseFailure("T-PLAN-RENDEZVOUS", f"tensor.imports.{conn.imp.get('name')}.rendezvous",
                                          f"missing outer events: {missing}"))
    return {r["event"]: r for r in conn.imp["rendezvous"]}


def plan_connection(name, export, imp, site, bindings=None, runtime=None):
    """-> the connection's record: routes tried in order with their outcomes, the certified
    program, what it reserves. Raises PipeLinkError (T-CONTRACT / T-MODEL / T-PLAN...) when no
    route is certified."""
    path = f"pipeline.tensor_connections.{name}"
    try:
        conn = Connection(export, imp, site, bindings, runtime)
    except Infeasible as why:
        raise PipeLinkError(ClauseFailure(why.clause, path, f"{why.outcome}: {why.reason}"))
    events = _rendezvous_events(conn)
    tried, chosen = [], None
    for route in ROUTE_ORDER:
        try:
            program = ROUTES[route](conn)
            used = certify(program, conn)
            used["barrier_generations"] += 2          # the outer ready and done events
            scratch, barrier = conn.lend("smem"), conn.lend("barrier")
            short = {}
            if used["scratch_bytes"] > (scratch or {}).get("extent", 0):
                short["smem_bytes"] = used["scratch_bytes"]
            if barrier is None or used["barrier_generations"] > (barrier.get("sync") or {}).get("generations", 0):
                short["barrier_generations"] = used["barrier_generations"]
            dest = conn.lend("reg", "dest")
            if dest is not None and dest["extent"] < len(conn.positions):
                short["dest_words"] = len(conn.positions)
            if short:
                raise Infeasible("RESOURCE_ENVELOPE", "the import's lends are too small for this route", facts=short)
            tried.append({"route": route, "outcome": "MODEL_SAT"})
            chosen = (route, program, used)
            break
        except Infeasible as why:
            # a route that does not apply, does not fit or does not lower is recorded and the next one
            # tried; inconsistent declarations and a missing frame end the planning
            if why.clause in ("T-MODEL", "T-CONTRACT", "T-PLAN-FRAME"):
                raise PipeLinkError(ClauseFailure(why.clause, path, f"{route}: {why.outcome}: {why.reason}", why.facts))
            tried.append({"route": route, "outcome": why.outcome, "reason": why.reason, **({"missing": why.facts} if why.facts else {})})
    if chosen is None:
        envelopes = [t for t in tried if t["outcome"] == "RESOURCE_ENVELOPE"]
        cheapest = envelopes[0] if envelopes else None
        raise PipeLinkError(ClauseFailure("T-PLAN", path, "no route fits the declared lends" if cheapest else "no route applies",
                                          {"tried": tried, **({"missing": cheapest.get("missing", {})} if cheapest else {})}))
    route, program, used = chosen
    scratch, barrier = conn.lend("smem"), conn.lend("barrier")
    claims = []
    if used["scratch_bytes"]:
        claims.append({"handle": scratch["location"]["handle"], "domain": "smem", "align": scratch.get("align", 16),
                       "extent": {"const": used["scratch_bytes"], "per": {}}})
    # a barrier lent at a link-time handle is claimed; one lent at a fixed id (location.base) is the consumer's own to keep free
    if barrier["location"].get("handle") is not None:
        claims.append({"handle": barrier["location"]["handle"], "domain": "named_barrier", "align": 1, "extent": {"const": 1, "per": {}}})
    text = json.dumps(program, sort_keys=True, separators=(",", ":"))
    return {"name": name, "export": export["name"], "import": imp["name"],
            # the adapter's symbol: a bare name, or the record {symbol, declaration, events, params} of the reference's units
            "callable": imp["callable"]["symbol"] if isinstance(imp["callable"], dict) else imp["callable"], "dtype": conn.dtype,
            "space": conn.space, "participants": len(conn.participants), "positions": len(conn.positions),
            "route_order": list(ROUTE_ORDER), "tried": tried, "route": route, "outcome": "MODEL_SAT", "program": program,
            "plan_sha256": hashlib.sha256(text.encode()).hexdigest(), "used": used, "claims": claims,
            "unused_handles": [scratch["location"]["handle"]] if scratch is not None and not used["scratch_bytes"] else [],
            "barrier_handle": barrier["location"].get("handle"), "barrier_id": barrier["location"].get("base"), "events": sorted(events),
            "coords": {"t": conn.t["name"], "p": conn.p["name"]}}


# ---------------------------------------------------------------- lowering
SOURCE_HEADER = "pipelink/tensor_source.h"


def _receipt_text(step, names, ctype, target):
    """tcgen05.ld 32x32b of `count` consecutive columns of the own lane, in chunks; then one wait."""
    out, done, count = [], 0, step["count"]
    col0 = expr_to_c(substitute(step["column"], {"i": ["const", 0]}), names)
    out.append(f"  const unsigned pl_taddr = pl_tmem + ((unsigned)(32 * ((threadIdx.x >> 5) & 3)) << 16) + (unsigned)({col0});")
    while done < count:
        n = next(c for c in RECEIPT_CHUNKS if c <= count - done)
        regs = ", ".join(f"%{k}" for k in range(n))
        outs = ", ".join(f'"=r"(pl_w[{done + k}])' for k in range(n))
        out.append(f'  asm volatile("tcgen05.ld.sync.aligned.32x32b.x{n}.b32 {{{regs}}}, [%{n}];" : {outs} : "r"(pl_taddr + {done}u) : "memory");')
        done += n
    out.append('  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");')
    if target == "dest":
        out.append(f"  #pragma unroll\n  for (int i = 0; i < {count}; ++i) dest[i] = {'__uint_as_float(pl_w[i])' if ctype == 'float' else f'({ctype})pl_w[i]'};")
    return out


def lower(record, *, warp_lo, threads_in_role):
    """CUDA text of one connection's adapter: `<fn>(source, dest, scratch)`, `<fn>_ready()`,
    `<fn>_done()`. Self-contained: it includes no stage header."""
    fn, ctype = record["callable"], C_TYPES[record["dtype"]]
    names = {record["coords"]["t"]: "pl_t", record["coords"]["p"]: "p", "i": "i"}
    tmem = record["space"] == "tmem"
    by_handle = record.get("barrier_handle") is not None
    bar = f"{record['barrier_handle']}()" if by_handle else f"{int(record.get('barrier_id') or 0)}"
    sync = [f'  asm volatile("bar.sync %0, %1;" :: "r"({bar}), "r"({threads_in_role}) : "memory");']
    if tmem:
        sync = ['  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");'] + sync + \
               ['  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");']
    L = [f"// connection {record['name']}: route {record['route']}, plan {record['plan_sha256'][:16]}",
         *([f'extern "C" __device__ int {record["barrier_handle"]}();'] if by_handle else []),
         f'extern "C" __device__ void {fn}_ready() {{', *sync, "}",
         f'extern "C" __device__ void {fn}_done() {{', *sync, "}",
         f'extern "C" __device__ void {fn}(pipelink_tensor_source source, {ctype}* dest, void* scratch) {{',
         f"  const int pl_t = (int)threadIdx.x - {32 * warp_lo};", "  (void)pl_t; (void)scratch;"]
    widest = max([s["count"] for s in record["program"] if s["op"] == "tmem_receipt"], default=0)
    if widest:
        L += [f"  unsigned pl_w[{widest}];", "  const unsigned pl_tmem = pipelink_source_tmem(source);"]
    for step in record["program"]:
        op = step["op"]
        if op == "tmem_receipt":
            L += _receipt_text(step, names, ctype, step["to"])
        elif op == "smem_store":
            L += [f"  #pragma unroll\n  for (int i = 0; i < {step['count']}; ++i) "
                  f"static_cast<unsigned*>(scratch)[{expr_to_c(step['word'], names)}] = pl_w[i];"]
        elif op == "rendezvous":
            L += sync[-2:-1] if tmem else sync
        elif op == "smem_load" and step["space"] == "scratch":
            L += [f"  #pragma unroll\n  for (int p = 0; p < {step['count']}; ++p) "
                  f"dest[p] = static_cast<const {ctype}*>(scratch)[{expr_to_c(step['word'], names)}];"]
        elif op == "smem_load":
            L += ["  const char* pl_src = static_cast<const char*>(pipelink_source_pointer(source));",
                  f"  #pragma unroll\n  for (int p = 0; p < {step['count']}; ++p) "
                  f"dest[p] = *reinterpret_cast<const {ctype}*>(pl_src + {expr_to_c(step['byte'], names)});"]
        elif op == "frame_load":
            L += [f"  const {ctype}* pl_frame = static_cast<const {ctype}*>(pipelink_source_pointer(source));",
                  f"  #pragma unroll\n  for (int p = 0; p < {step['count']}; ++p) dest[p] = pl_frame[{expr_to_c(step['index'], names)}];"]
    L.append("}")
    return "\n".join(L) + "\n"


def adapters_unit(records, roles):
    """One generated translation unit with every connection's adapter. roles: role name ->
    (warp_lo, warps) of the consumer site's role."""
    text = ["// generated by pipec2 link: tensor import adapters", "#include <cuda_runtime.h>", f"#include <{SOURCE_HEADER}>", ""]
    for rec in records:
        warp_lo, warps = roles[rec["site_role"]]
        if rec["space"] == "tmem" and (warp_lo % 4 != 0):
            raise PipeLinkError(ClauseFailure("T-LOWER", f"pipeline.tensor_connections.{rec['name']}",
                                              f"role {rec['site_role']!r} starts at warp {warp_lo}: tensor-memory receipt needs a multiple of four"))
        text.append(lower(rec, warp_lo=warp_lo, threads_in_role=32 * warps))
    return "\n".join(text)


# ---------------------------------------------------------------- all connections of a pipeline
def plan_pipeline(manifests, pipe):
    """Plan every entry of the pipeline's `tensor_connections`:
    {"name", "producer", "export", "consumer", "import"}. -> records (each with `consumer`,
    `site_role` and the claims to merge into the consumer's)."""
    by_id = {m["stage"]["id"]: m for m in manifests}
    records, fed = [], {}
    for c in pipe.get("tensor_connections", []):
        path = f"pipeline.tensor_connections.{c.get('name')}"
        if "producer" not in c and "consumer" not in c:        # the reference's spelling: "stage id:export", "stage id:import"
            c = dict(c)
            c["producer"], _, c["export"] = str(c.get("export", "")).rpartition(":")
            c["consumer"], _, c["import"] = str(c.get("import", "")).rpartition(":")
        prod, cons = by_id.get(c.get("producer")), by_id.get(c.get("consumer"))
        if prod is None or cons is None:
            raise PipeLinkError(ClauseFailure("T-CONTRACT", path, "producer or consumer is not a stage of the pipeline"))
        export = next((e for e in (prod.get("tensor") or {}).get("exports", []) if e["name"] == c.get("export")), None)
        imp = next((i for i in (cons.get("tensor") or {}).get("imports", []) if i["name"] == c.get("import")), None)
        if export is None or imp is None:
            raise PipeLinkError(ClauseFailure("T-CONTRACT", path, "the named export or import is not declared"))
        # one export feeds several imports only when they are independent; this build admits one
        if (c["producer"], c["export"]) in fed:
            raise PipeLinkError(ClauseFailure("T-CONTRACT", path, f"export already feeds {fed[(c['producer'], c['export'])]!r}: dependent fanout"))
        fed[(c["producer"], c["export"])] = c["name"]
        site_name = (imp.get("sites") or [None])[0]
        site = dict(next((s for s in (cons.get("tensor") or {}).get("sites", []) if s["name"] == site_name), {}))
        role = site.get("role")
        if role not in cons["stage"]["roles"]:
            raise PipeLinkError(ClauseFailure("T-CONTRACT", path, f"site {site_name!r} names no role of the consumer"))
        site["participants"] = 32 * cons["stage"]["roles"][role]["warps"]
        site["warpgroup_aligned"] = any(cl.get("domain") == "warp" and role in cl.get("roles", []) and cl.get("align", 1) % 4 == 0
                                        for cl in cons.get("claims", []))
        declared = (prod.get("tensor") or {}).get("bindings", [])
        binds = {b["name"]: b["domain"]["values"][0] for b in declared if len(b.get("domain", {}).get("values", [])) == 1}
        runtime = {b["name"]: {"values": list(b["domain"]["values"]), "units": b.get("units")} for b in declared
                   if len(b.get("domain", {}).get("values", [])) > 1}
        # the only role of the pipeline that owns warps starts at warp 0, whatever its claim's alignment
        owners = [r for m in manifests for r, spec in m["stage"]["roles"].items() if spec.get("warps", 0) > 0]
        site["warpgroup_aligned"] = site["warpgroup_aligned"] or owners == [role]
        rec = plan_connection(c["name"], export, imp, site, binds, runtime)
        rec.update(producer=c["producer"], consumer=c["consumer"], site_role=role)
        records.append(rec)
    return records
