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


def pair_channels(manifests: list[dict]):
    """-> {channel: (producer (stage_id, endpoint), consumer (stage_id, endpoint))}"""
    by_name = {}
    for m in manifests:
        for ep in m.get("endpoints", []):
            by_name.setdefault(ep["name"], []).append((m["stage"]["id"], ep))
    failures, channels = [], {}
    for name, eps in sorted(by_name.items()):
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


def expand_protocols(channels, manifests) -> list[dict]:
    """One expansion record per channel: barrier slot handles, arrival counts, tx bytes, depth."""
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
                if count not in legal:
                    failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol.{side}.arrive.count",
                                                  f"{count} arrivals cannot come from role {by!r} ({warps[by]} warps)",
                                                  {"legal": sorted(legal)}))
                rec[side] = {"slots": s["slots"], "count": count, "by": by, "tx_bytes": s.get("tx_bytes", 0)}
            full = proto.get("full") or {}
            if full.get("tx_bytes", 0) not in (0, ring.get("stage_stride_bytes", 0)) and pe["proxy"] == "async" and pe["space"] == "smem":
                failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol.full.tx_bytes",
                                              "expected transaction bytes differ from the ring's stage stride"))
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
