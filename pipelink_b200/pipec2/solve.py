"""Link-time resource solve with Z3: ring depths, claim bases per domain, warp tiling.

Same problem statement as the reference's solver (pipec/src/pipec2/solve.py:815-1007; objective
order docs/reference/pack-and-link.md:131-141): one integer per bindable depth handle (from its
candidate values) and one per claim base; claims in domains that share a physical resource must
not overlap (an mbarrier slot occupies 16 bytes of shared memory); bases respect alignment,
granularity, absolute placement and the domain capacity; role warp claims tile ``[0, warps)``
exactly. Objective, lexicographic: maximise depths in priority order, then minimise the
high-water mark of each physical domain. Unsatisfiable problems are reported with the clause
whose constraints were in the unsat core, by the reference's precedence
``L-OVERLAP > L-HANDLE > L-TOPO > L-ALIGN`` (solve.py:494,603-627).
"""
from __future__ import annotations

import z3

from .model import ClauseFailure, PipeLinkError

SOLVE_TIMEOUT_MS = 120000
PRECEDENCE = ("L-BUDGET", "L-OVERLAP", "L-HANDLE", "L-TOPO", "L-ALIGN", "L-REGS")


def _extent_expr(extent, depth_vars):
    e = extent.get("const", 0)
    for handle, coef in extent.get("per", {}).items():
        e = e + coef * depth_vars[handle]
    return e


def solve(claims: dict, handles: dict, profile: dict, *, depth_priority=(), forced=None, total_warps=None,
          regs_priority=(), reg_claims=(), role_warps=None, pipeline_domains=None, exclusive=()):
    """claims: handle -> unified claim record (every domain but `regs`). reg_claims: the register
    claims ({handle, roles, values, reg_group?}); role_warps: role -> (warp claim handle, warps[, offset inside the claim]).
    Returns (bindings, intervals, tiers)."""
    forced = forced or {}
    pipeline_domains = pipeline_domains or {}
    opt = z3.Optimize()
    opt.set(priority="lex")
    tracked = []  # (bool, clause, path) for diagnostics through a parallel Solver
    cons = []

    def add(expr, clause, path):
        cons.append((expr, clause, path))

    depth_vars = {}
    for name, h in handles.items():
        if h["class"] != "depth":
            continue
        v = z3.Int(name)
        depth_vars[name] = v
        values = [forced[name]] if name in forced else h["values"]
        if name in forced and forced[name] not in h["values"]:
            raise PipeLinkError(ClauseFailure("L-HANDLE", f"pipeline.forced_bindings.{name}",
                                              f"{forced[name]} is not a candidate value", {"values": h["values"]}))
        add(z3.Or([v == x for x in values]), "L-HANDLE", f"handles.{name}.values")

    base_vars, ext_exprs = {}, {}
    domains = dict(profile["domains"])
    for dname, dom in list(domains.items()):
        if dom.capacity == "pipeline":      # the pipeline description sizes this domain (0 when it does not)
            stated = pipeline_domains.get(dname) or {}
            cap = int(stated.get("capacity", 0))
            domains[dname] = type(dom)(dom.unit, cap, dom.lowest, dom.granularity, dom.physical, int(stated.get("page_bytes", dom.scale)))
    for name, cl in claims.items():
        dom = domains[cl["domain"]]
        b = z3.Int(name)
        base_vars[name] = b
        ext = _extent_expr(cl["extent"], depth_vars)
        gran = max(dom.granularity, 1)
        # the domain granularity constrains where a claim may start, not how long it is (the
        # reference places 24 scale columns at [128, 152), pipec/src/pipec2/solve.py)
        ext_g = ext
        ext_exprs[name] = ext_g
        # a claim that cannot be placed inside its domain is a placement failure like any other: the reference
        # tracks the capacity of a domain under L-OVERLAP, path solve.capacity.<domain> (pipec/src/pipec2/solve.py);
        # L-BUDGET is kept for a solve that runs out of its allowance
        add(b >= dom.lowest, "L-OVERLAP", f"solve.capacity.{dom.physical}")
        add(b + ext_g <= dom.capacity + dom.lowest, "L-OVERLAP", f"solve.capacity.{dom.physical}")
        align = max(cl.get("align", 1), gran)
        if align > 1:
            add(b % align == 0, "L-ALIGN", f"claims.{name}.align")
        if "absolute_base" in cl:
            add(b == cl["absolute_base"], "L-ALIGN", f"claims.{name}.absolute_base")
        if name in forced:
            add(b == forced[name], "L-HANDLE", f"pipeline.forced_bindings.{name}")

    # non-overlap inside every physical resource (kernel-lifetime claims only in this build). Shared
    # memory holds the many small claims (every barrier slot array is one): there the claims that
    # nothing pins are laid out in one fixed order, strictest alignment first, each behind the last,
    # which needs no disjunctions and packs as tightly as any order does when alignments decrease;
    # pinned claims (a forced or absolute base) and the small domains keep pairwise exclusion.
    names = sorted(claims)

    def may_share(a, bname):
        """Two claims that live in phases the pipeline declares exclusive are never live together: they
        may occupy the same space (the reference's phase lifetimes, docs/reference/annotations.md:294-300)."""
        la, lb = claims[a].get("lifetime", "kernel"), claims[bname].get("lifetime", "kernel")
        if not (isinstance(la, str) and isinstance(lb, str) and la.startswith("phase:") and lb.startswith("phase:")):
            return False
        x, y = la[len("phase:"):], lb[len("phase:"):]
        from fnmatch import fnmatchcase
        return x != y and any((fnmatchcase(x, p) and fnmatchcase(y, q)) or (fnmatchcase(x, q) and fnmatchcase(y, p))
                              for p, q in exclusive)

    def span(n):
        d = domains[claims[n]["domain"]]
        return base_vars[n] * d.scale, (base_vars[n] + ext_exprs[n]) * d.scale

    def exclude(a, bname):
        (lo_a, hi_a), (lo_b, hi_b) = span(a), span(bname)
        add(z3.Or(hi_a <= lo_b, hi_b <= lo_a), "L-OVERLAP", f"claims.{a}~{bname}")

    for phys in sorted({d.physical for d in domains.values()}):
        members = [n for n in names if domains[claims[n]["domain"]].physical == phys]
        pinned = [n for n in members if n in forced or "absolute_base" in claims[n] or
                  str(claims[n].get("lifetime", "kernel")).startswith("phase:")]
        free = [n for n in members if n not in pinned]
        if phys == "smem" and len(free) > 2:
            byte_align = lambda n: max(claims[n].get("align", 1), 1) * domains[claims[n]["domain"]].scale
            free.sort(key=lambda n: (-byte_align(n), n))
            for prev, nxt in zip(free, free[1:]):
                add(span(prev)[1] <= span(nxt)[0], "L-OVERLAP", f"claims.{prev}~{nxt}")
            for a in pinned:
                for bname in members:
                    if bname != a and (bname not in pinned or a < bname) and not may_share(a, bname):
                        exclude(a, bname)
        else:
            for i, a in enumerate(members):
                for bname in members[i + 1:]:
                    if not may_share(a, bname):
                        exclude(a, bname)

    # warp claims tile [0, total) exactly
    warp_claims = [n for n in names if claims[n]["domain"] == "warp"]
    if warp_claims:
        total = sum(claims[n]["extent"]["const"] for n in warp_claims)
        for n in warp_claims:
            add(base_vars[n] + claims[n]["extent"]["const"] <= total, "L-TOPO", f"claims.{n}.warp_tiling")
        if total > domains["warp"].capacity:
            raise PipeLinkError(ClauseFailure("L-TOPO", "topology.warps", f"{total} warps exceed the launch limit"))

    # register groups (pipec/src/pipec2/solve.py:737-812): every group is a run of whole warpgroups
    # that contains exactly its member roles; the chosen per-thread counts must fit the register
    # file the launch is given (launch threads x the launch's per-thread allocation)
    regs_vars, reg_groups = {}, []
    caps = profile.get("caps", {})
    if reg_claims:
        path = "solve.register_groups"
        role_warps = role_warps or {}
        wg = caps.get("warpgroup_warps", 4)
        assigned, pool = set(), 0
        launch_threads = 32 * sum(rw[1] for rw in role_warps.values())
        for cl in sorted(reg_claims, key=lambda c: c["handle"]):
            name = cl.get("reg_group") or (cl["roles"][0] if len(cl["roles"]) == 1 else None)
            h = handles.get(cl["handle"])
            members = sorted(set(cl["roles"]))
            bad = (name is None or h is None or h.get("class") != "regs" or h.get("domain") != "regs" or
                   h.get("owner") != f"reg_group:{name}" or not members or
                   any(r in assigned or r not in role_warps for r in members))
            if bad:
                add(z3.BoolVal(False), "L-REGS", path)
                continue
            assigned.update(members)
            v = z3.Int(cl["handle"])
            regs_vars[cl["handle"]] = v
            values = [forced[cl["handle"]]] if cl["handle"] in forced else sorted(set(h["values"]) & set(cl["values"]))
            add(z3.Or([v == x for x in values]) if values else z3.BoolVal(False), "L-REGS", path)
            width = sum(role_warps[r][1] for r in members)
            lo = z3.Int(f"reg_group:{name}:lo")
            add(z3.And(lo >= 0, lo % wg == 0, (lo + width) % wg == 0), "L-REGS", path)
            for r in members:
                rb = base_vars[role_warps[r][0]] + (role_warps[r][2] if len(role_warps[r]) > 2 else 0)
                add(z3.And(rb >= lo, rb + role_warps[r][1] <= lo + width), "L-REGS", path)
            pool = pool + v * width * 32
            reg_groups.append({"name": name, "handle": cl["handle"], "roles": members, "lo": lo, "width": width})
        if assigned != set(role_warps):
            add(z3.BoolVal(False), "L-REGS", path)
        expected = {n for n, h in handles.items() if h.get("class") == "regs"}
        if expected != set(regs_vars):
            add(z3.BoolVal(False), "L-REGS", path)
        gran = caps.get("reg_alloc_granularity", 8)
        launch_regs = z3.Int("__launch_regs")
        add(z3.And(launch_regs % gran == 0, launch_regs >= caps.get("regs_min", 24), launch_regs <= caps.get("regs_max", 255),
                   launch_regs * launch_threads <= caps.get("regs_per_sm", 65536), pool <= launch_regs * launch_threads),
            "L-REGS", path)
    elif any(h.get("class") == "regs" for h in handles.values()):
        # no role asks for registers of its own: the one register handle an image may then carry is the
        # launch allocation itself (owner reg_group:launch): one count for every thread, taken from the
        # handle's values, as large as the register file allows for the launch's threads
        launch = [n for n, h in handles.items() if h.get("class") == "regs"]
        h = handles[launch[0]]
        launch_threads = 32 * sum(rw[1] for rw in (role_warps or {}).values())
        if len(launch) != 1 or h.get("owner") != "reg_group:launch" or h.get("domain") != "regs" or not launch_threads:
            add(z3.BoolVal(False), "L-REGS", "solve.register_groups")
        else:
            v = z3.Int(launch[0])
            regs_vars[launch[0]] = v
            values = [forced[launch[0]]] if launch[0] in forced else sorted(h["values"])
            add(z3.Or([v == x for x in values]), "L-REGS", "solve.register_groups")
            add(z3.And(v >= caps.get("regs_min", 24), v <= caps.get("regs_max", 255),
                       v * launch_threads <= caps.get("regs_per_sm", 65536)), "L-REGS", "solve.register_groups")

    for expr, _, _ in cons:
        opt.add(expr)

    tiers = []
    for name in depth_priority:
        if name in depth_vars:
            opt.maximize(depth_vars[name])
            tiers.append({"name": f"max {name}"})
    for name in sorted(depth_vars):
        if name not in depth_priority:
            opt.maximize(depth_vars[name])
            tiers.append({"name": f"max {name}"})
    for name in list(regs_priority) + sorted(n for n in regs_vars if n not in regs_priority):
        if name in regs_vars:
            opt.maximize(regs_vars[name])
            tiers.append({"name": f"max {name}"})
    if reg_claims:
        opt.minimize(z3.Int("__launch_regs"))       # the smallest launch allocation that covers the pool
        tiers.append({"name": "min launch registers"})
    highwater = {}
    for phys in sorted({d.physical for d in domains.values()}):
        members = [n for n in names if domains[claims[n]["domain"]].physical == phys]
        if not members:
            continue
        hw = z3.Int(f"__hw_{phys}")
        for n in members:
            opt.add(hw >= (base_vars[n] + ext_exprs[n]) * domains[claims[n]["domain"]].scale)
        highwater[phys] = hw
        opt.minimize(hw)
        tiers.append({"name": f"min high-water {phys}"})
    # finally prefer low bases so layouts are deterministic
    for n in names:
        opt.minimize(base_vars[n])

    opt.set("timeout", SOLVE_TIMEOUT_MS)
    verdict = opt.check()
    if verdict == z3.unknown:       # a link must end: say so instead of searching on
        raise PipeLinkError(ClauseFailure("L-BUDGET", "solve", f"the solver gave up after {SOLVE_TIMEOUT_MS // 1000} s "
                                          f"({opt.reason_unknown()}); pin some bases in forced_bindings or declare fewer claims"))
    if verdict != z3.sat:
        _diagnose(cons)
    model = opt.model()
    val = lambda e: e if isinstance(e, int) else model.eval(e, model_completion=True).as_long()
    bindings = {n: [val(v), "forced" if n in forced else "solved"] for n, v in depth_vars.items()}
    intervals = {}
    for n in names:
        lo = val(base_vars[n])
        hi = lo + val(ext_exprs[n])
        bindings[n] = [lo, "forced" if n in forced else "solved"]
        intervals.setdefault(claims[n]["domain"], []).append(
            {"handle": n, "lo": lo, "hi": hi, "phase": claims[n].get("lifetime", "kernel")})
    for tier in tiers:
        tier["status"] = "optimal"
    hw_vals = {phys: val(hw) for phys, hw in highwater.items()}
    info = {"tiers": tiers, "high_water": hw_vals, "engine": f"z3 {z3.get_version_string()} Optimize(lex)"}
    if not reg_claims and regs_vars:
        (n, v), = regs_vars.items()
        bindings[n] = [val(v), "forced" if n in forced else "solved"]
        info["launch_regs"] = val(v)
    if reg_claims:
        for n, v in regs_vars.items():
            bindings[n] = [val(v), "forced" if n in forced else "solved"]
        info["launch_regs"] = val(z3.Int("__launch_regs"))
        info["reg_groups"] = [{"name": g["name"], "handle": g["handle"], "roles": g["roles"], "warp_lo": val(g["lo"]),
                               "warp_hi": val(g["lo"]) + g["width"], "regs": val(regs_vars[g["handle"]])} for g in reg_groups]
    return bindings, intervals, info


def _diagnose(cons):
    """Map an unsatisfiable problem to clause failures through a tracked unsat core."""
    s = z3.Solver()
    labels = {}
    for i, (expr, clause, path) in enumerate(cons):
        p = z3.Bool(f"c{i}")
        labels[str(p)] = (clause, path)
        s.assert_and_track(expr, p)
    failures = [ClauseFailure("L-BUDGET", "solve", "no assignment satisfies the resource constraints")]
    if s.check() == z3.unsat:
        core = [labels[str(c)] for c in s.unsat_core()]
        best = min((PRECEDENCE.index(c) if c in PRECEDENCE else 99) for c, _ in core)
        clause = PRECEDENCE[best] if best < len(PRECEDENCE) else core[0][0]
        failures = [ClauseFailure(clause, path, "constraint is part of the unsatisfiable core") for c, path in core if c == clause]
    raise PipeLinkError(failures)
