"""Cross-stage contract checks: endpoint pairing, physical layout identity, protocol expansion.

Follows the reference's link phases (pipec/src/pipec2/link.py:1614-1700: ``_pair_channels`` ->
``_canonical_endpoints`` / ``_unify_pairs`` (clause L8) -> ``protocol.expand``,
pipec/src/pipec2/protocol.py:92-110,511-640): a channel is one ``produce`` and one ``consume``
endpoint of the same name; both must state the same space, scope, proxy, tile, canonical layout,
ring and protocol; arrive counts are checked against the arriving role's size.
"""
from __future__ import annotations

from .model import ClauseFailure, PipeLinkError

COMPAT_FIELDS = ("space", "scope", "proxy", "tile", "binds")


def canonical_layout(layout: dict | None):
    """Flatten nested modes, drop unit modes and merge contiguous ones; keep the swizzle.
    Tensor-memory layouts are `lanes` [start, stop) and `cols` (pipec/src/pipec2/layout.py:75-78)."""
    if layout is None:
        return None
    if "lanes" in layout or "cols" in layout:   # tensor memory: a lane range and a column count
        return {"elem_bits": layout.get("elem_bits"), "lanes": list(layout.get("lanes", ())), "cols": layout.get("cols")}
    shape = [s for mode in layout["shape"] for s in mode]
    stride = [s for mode in layout["stride"] for s in mode]
    modes = [(sh, st) for sh, st in zip(shape, stride) if sh != 1]
    merged = []
    for sh, st in reversed(modes):           # innermost first
        if merged and merged[-1][1] * merged[-1][0] == st:
            merged[-1] = (merged[-1][0] * sh, merged[-1][1])
        else:
            merged.append((sh, st))
    return {"elem_bits": layout.get("elem_bits"), "modes": list(reversed(merged)),
            "swizzle": layout.get("swizzle")}


def _by_name(manifests):
    by_name = {}
    for m in manifests:
        for ep in m.get("endpoints", []):
            by_name.setdefault(ep["name"], []).append((m["stage"]["id"], ep))
    return by_name


def _is_counter(eps) -> bool:
    return any((e[1].get("protocol") or {}).get("kind") == "counter" for e in eps)


def counter_channels(manifests: list[dict]):
    """Counter channels: one or more producers and any number of consumers, across stages
    (docs/reference/annotations.md:217-237). -> {channel: (producers, consumers)}; a consumer
    without a producer is an L-PAIR failure."""
    failures, out = [], {}
    for name, eps in sorted(_by_name(manifests).items()):
        if not _is_counter(eps):
            continue
        prod = [e for e in eps if e[1]["direction"] == "produce"]
        cons = [e for e in eps if e[1]["direction"] == "consume"]
        if not prod:
            failures.append(ClauseFailure("L-PAIR", f"channels.{name}", "a counter channel needs at least one producer"))
            continue
        out[name] = (prod, cons)
    if failures:
        raise PipeLinkError(failures)
    return out


def expand_counters(counters, handles) -> list[dict]:
    """One record per counter channel: `counter` = [slot handle, release operation, sorted acquire
    patterns] (pipec/src/pipec2/protocol.py:821-853). Every endpoint agrees on scope, slot and
    release; each consumer chooses its own acquire pattern."""
    releases = {"grid": "red.release.gpu", "system": "red.release.sys"}
    acquires = {"grid": ("ld.acquire.gpu", "ld.relaxed.gpu+fence.acquire.gpu"),
                "system": ("ld.acquire.sys", "ld.relaxed.sys+fence.acquire.sys")}
    failures, out = [], []
    for name, (prod, cons) in sorted(counters.items()):
        path = f"channels.{name}.protocol"
        eps = [e for _, e in prod + cons]
        decls = [(e.get("protocol") or {}).get("counter") for e in eps]
        if any(e.get("protocol", {}).get("kind") != "counter" or d is None for e, d in zip(eps, decls)):
            failures.append(ClauseFailure("L-PROTO", path, "counter channel needs a counter declaration on every endpoint"))
            continue
        first = decls[0]
        h = handles.get(first["slot"])
        if h is None or h.get("class") != "base" or h.get("domain") != "gmem_counter":
            failures.append(ClauseFailure("L-PROTO", path, "counter slot handle is not declared in the gmem_counter domain"))
            continue
        if any(e.get("space") != "gmem" for e in eps):
            failures.append(ClauseFailure("L-PROTO", path, "counter channels must use gmem space"))
            continue
        scope = eps[0].get("scope")
        if scope not in releases:
            failures.append(ClauseFailure("L-PROTO", f"{path}.scope", "a counter is grid- or system-scoped"))
            continue
        agreed = (scope, first["slot"], first.get("release", releases[scope]))
        if any((e.get("scope"), d["slot"], d.get("release", releases[scope])) != agreed for e, d in zip(eps, decls)):
            failures.append(ClauseFailure("L-PROTO", path, "counter scope, slot or release operation disagree"))
            continue
        if agreed[2] != releases[scope]:
            failures.append(ClauseFailure("L-PROTO", f"{path}.release", f"a {scope}-scoped counter is released with {releases[scope]}"))
            continue
        acq = sorted({d.get("acquire", acquires[scope][0]) for (_, e), d in zip(prod + cons, decls) if e["direction"] == "consume"})
        if any(a not in acquires[scope] for a in acq):
            failures.append(ClauseFailure("L-PROTO", f"{path}.acquire", "acquire pattern outside the scope's vocabulary"))
            continue
        out.append({"channel": name, "kind": "counter", "producers": sorted(s for s, _ in prod),
                    "consumers": sorted(s for s, _ in cons), "counter": [first["slot"], agreed[2], acq]})
    if failures:
        raise PipeLinkError(failures)
    return out


def check_topology(manifests, profile):
    """All stages of one image agree on the CTA group and on the compiled cluster shape
    (clause L-TOPO; the reference intersects the same declarations, pipec/src/pipec2/link.py:1040-1100)."""
    failures = []
    groups = {m["stage"]["id"]: (m.get("topology", {}).get("cta_group") or {}).get("fixed", 1) for m in manifests}
    clusters = {m["stage"]["id"]: tuple((m.get("topology", {}).get("cluster") or {}).get("compiled", [1, 1, 1])) for m in manifests}
    if len(set(groups.values())) > 1:
        failures.append(ClauseFailure("L-TOPO", "stages.topology.cta_group", "stages were compiled for different CTA groups", {"stages": groups}))
    if len(set(clusters.values())) > 1:
        failures.append(ClauseFailure("L-TOPO", "stages.topology.cluster.compiled", "stages were compiled for different cluster shapes",
                                      {"stages": {k: list(v) for k, v in clusters.items()}}))
    if failures:
        raise PipeLinkError(failures)
    group, cluster = next(iter(groups.values())), next(iter(clusters.values()))
    caps = profile.get("caps", {})
    if group not in caps.get("cta_group_legal", (1,)):
        raise PipeLinkError(ClauseFailure("L-TOPO", "topology.cta_group", f"CTA group {group} is not legal on this target"))
    if any(c < 1 or c > mx for c, mx in zip(cluster, caps.get("max_cluster", (1, 1, 1)))):
        raise PipeLinkError(ClauseFailure("L-TOPO", "topology.cluster.compiled", f"cluster {list(cluster)} exceeds the target's limit"))
    size = cluster[0] * cluster[1] * cluster[2]
    if group == 2 and size % 2:
        raise PipeLinkError(ClauseFailure("L-TOPO", "topology.cluster.compiled", "a CTA pair needs an even cluster"))
    return group, cluster


def pair_channels(manifests: list[dict]):
    """-> {channel: (producer (stage_id, endpoint), consumer (stage_id, endpoint))} for every channel
    that pairs exactly one producer with one consumer (all protocols but counters)."""
    failures, channels = [], {}
    for name, eps in sorted(_by_name(manifests).items()):
        if _is_counter(eps):
            continue
        prod = [e for e in eps if e[1]["direction"] == "produce"]
        cons = [e for e in eps if e[1]["direction"] == "consume"]
        if len(prod) != 1 or len(cons) != 1:
            failures.append(ClauseFailure("L-PAIR", f"channels.{name}",
                                          f"needs exactly one producer and one consumer, found {len(prod)} and {len(cons)}"))
            continue
        channels[name] = (prod[0], cons[0])
    if failures:
        raise PipeLinkError(failures)
    return channels


def physical_identity(ep: dict):
    """What both ends of a channel must agree on byte for byte: the canonical layout and how far
    apart ring stages are (the reference's `endpoint.physical_identity`, clause L8)."""
    return {"layout": canonical_layout(ep.get("layout")), "stage_stride_bytes": (ep.get("ring") or {}).get("stage_stride_bytes")}


def check_compatibility(channels) -> None:
    failures = []
    for name, ((ps, pe), (cs, ce)) in channels.items():
        for stage, ep in ((ps, pe), (cs, ce)):
            lay = ep.get("layout") or {}
            if ep.get("space") == "tmem" and "lanes" in lay:
                lanes = lay["lanes"][1] - lay["lanes"][0]
                if [lanes, lay.get("cols")] != list(ep.get("tile", {}).get("shape", [])):
                    failures.append(ClauseFailure("L8", f"endpoints.{name}.layout",
                                                  "TMEM lane/column shape is not congruent with tile.shape", {"stage": stage}))
        if failures:
            continue
        for f in COMPAT_FIELDS:
            if pe.get(f) != ce.get(f):
                failures.append(ClauseFailure("L-PAIR", f"channels.{name}.endpoint.{f}",
                                              f"endpoint compatibility field {f} differs",
                                              {"producer": ps, "consumer": cs}))
        if (pe.get("ring") or {}).get("depth") != (ce.get("ring") or {}).get("depth"):
            failures.append(ClauseFailure("L-PAIR", f"channels.{name}.endpoint.ring", "ring depths differ",
                                          {"producer": ps, "consumer": cs}))
        if physical_identity(pe) != physical_identity(ce):
            failures.append(ClauseFailure("L8", f"channels.{name}.layout", "paired endpoints describe different physical layouts",
                                          {"producer": physical_identity(pe), "consumer": physical_identity(ce)}))
        if pe.get("protocol") != ce.get("protocol"):
            failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol", "endpoint protocols differ"))
    if failures:
        raise PipeLinkError(failures)


def _role_sizes(manifests):
    sizes = {}
    for m in manifests:
        for role, r in m["stage"]["roles"].items():
            sizes[role] = r["warps"]
    return sizes


def expand_protocols(channels, manifests, cluster_size: int = 1) -> list[dict]:
    """One expansion record per channel: barrier slot handles, arrival counts, tx bytes, depth.
    A cluster-scoped channel may collect its arrivals from the role's warps in every CTA of the
    cluster (the reference's example: pl::side{..., {"producer", 2}, 0} under .scope("cluster"),
    docs/reference/annotations.md:205-209)."""
    warps = _role_sizes(manifests)
    failures, out = [], []
    for name, ((ps, pe), (cs, ce)) in sorted(channels.items()):
        proto = pe["protocol"]
        ring = pe.get("ring", {})
        depth = ring.get("depth")
        rec = {"channel": name, "kind": proto["kind"], "producer": ps, "consumer": cs,
               "depth": depth, "stage_stride_bytes": ring.get("stage_stride_bytes", 0)}
        if proto["kind"] == "mbarrier":
            for side in ("full", "empty"):
                s = proto.get(side)
                if s is None:
                    rec[side] = None
                    continue
                by, count = s["arrive"]["by"], s["arrive"]["count"]
                if by not in warps:
                    failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol.{side}.arrive.by", f"unknown role {by!r}"))
                    continue
                legal = {1, warps[by], 32 * warps[by]}
                if pe.get("scope") == "cluster":
                    legal |= {cluster_size * n for n in (1, warps[by], 32 * warps[by])}
                if count not in legal:
                    failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol.{side}.arrive.count",
                                                  f"{count} arrivals cannot come from role {by!r} ({warps[by]} warps)",
                                                  {"legal": sorted(legal)}))
                rec[side] = {"slots": s["slots"], "count": count, "by": by, "tx_bytes": s.get("tx_bytes", 0)}
            full = proto.get("full") or {}
            tx, stride = full.get("tx_bytes", 0), ring.get("stage_stride_bytes", 0)
            # a slot may carry padding behind its payload (alignment of the next slot), never less than it
            payload = ring.get("payload_bytes", stride)
            if tx not in (0, payload, cluster_size * payload) and pe["proxy"] == "async" and pe["space"] == "smem":
                failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol.full.tx_bytes",
                                              "expected transaction bytes differ from the ring slot's payload"))
            if payload > stride:
                failures.append(ClauseFailure("L-PROTO", f"channels.{name}.ring.payload_bytes", "a slot's payload exceeds its stride"))
            init = proto.get("init", {})
            if init.get("materializer") != "dispatch":
                failures.append(ClauseFailure("L-OWNER", f"channels.{name}.protocol.init", "barrier init needs a single materializer (dispatch)"))
            rec["init"] = init
        elif proto["kind"] == "call":
            rec["callable"] = [proto["export"], proto.get("decl", "")]
        else:
            failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol.kind", f"unsupported protocol kind {proto['kind']!r}"))
        out.append(rec)
    if failures:
        raise PipeLinkError(failures)
    return out
