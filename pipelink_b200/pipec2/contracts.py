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
    flat = lambda modes: [s for mode in modes for s in (mode if isinstance(mode, (list, tuple)) else [mode])]
    shape, stride = flat(layout["shape"]), flat(layout["stride"])
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
        # the declaration sits in `protocol.counter`, or flat in the protocol (the form the reference's annotation pass emits)
        def declaration(e):
            proto = e.get("protocol") or {}
            if proto.get("counter") is not None:
                return proto["counter"]
            return {k: proto[k] for k in ("slot", "release", "acquire") if k in proto} if "slot" in proto else None

        decls = [declaration(e) for e in eps]
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


def check_topology(manifests, profile, pipeline_topology=None):
    """All stages of one image agree on the CTA group and on the compiled cluster shape, and with the
    pipeline on whether the kernel is persistent and who schedules it
    (clause L-TOPO; the reference intersects the same declarations, pipec/src/pipec2/link.py:1040-1100)."""
    failures = []
    for m in manifests:
        for key in ("persistent", "scheduler"):
            mine, theirs = m.get("topology", {}).get(key), (pipeline_topology or {}).get(key)
            if mine is not None and theirs is not None and mine != theirs:
                failures.append(ClauseFailure("L-TOPO", f"stages.{m['stage']['id']}.topology.{key}",
                                              f"the stage was written for {key} = {mine!r}, the pipeline states {theirs!r}"))
    groups = {m["stage"]["id"]: (m.get("topology", {}).get("cta_group") or {}).get("fixed", 1) for m in manifests}
    def compiled(m):
        # "dynamic": the stage was compiled without a cluster attribute; the launch chooses (one CTA here)
        c = (m.get("topology", {}).get("cluster") or {}).get("compiled", [1, 1, 1])
        return (1, 1, 1) if c == "dynamic" else tuple(c)

    clusters = {m["stage"]["id"]: compiled(m) for m in manifests}
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
        handoff = (pe.get("protocol") or {}).get("kind") == "named_barrier"
        for f in COMPAT_FIELDS:
            # the two ends of a named-barrier hand-off may hold the handed-over storage under claims of
            # their own (one per phase); that the claims are the same place is checked once they are solved
            if handoff and f == "binds":
                continue
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
        failures += _protocol_differences(name, pe.get("protocol") or {}, ce.get("protocol") or {})
    if failures:
        raise PipeLinkError(failures)


def _protocol_differences(name, pp, cp):
    """Where the two ends of a channel state their protocol differently, most specific path first
    (the reference reports e.g. `channels.<name>.protocol.full.arrive`, pipec/src/pipec2/protocol.py:560-640)."""
    path = f"channels.{name}.protocol"
    if pp.get("kind") != cp.get("kind"):
        return [ClauseFailure("L-PROTO", f"{path}.kind", "endpoint protocol kinds differ")]
    if pp.get("kind") == "named_barrier":
        # a hardware named barrier both roles reach: the ends name the same id handle and thread count
        if (pp.get("id"), pp.get("count")) != (cp.get("id"), cp.get("count")):
            return [ClauseFailure("L-PROTO", path, "named-barrier id handle or thread count disagrees")]
        return []
    if pp.get("kind") == "call":
        # the two ends declare different functions by design (trampoline / implementation); they agree on
        # the export they mean and on its signature
        if (pp.get("export"), pp.get("signature")) != (cp.get("export"), cp.get("signature")):
            return [ClauseFailure("L-PROTO", path, "caller and provider disagree on the export or its signature")]
        return []
    out = []
    for side in ("full", "empty"):
        ps, cs = pp.get(side) or {}, cp.get(side) or {}
        if ps.get("arrive") != cs.get("arrive"):
            out.append(ClauseFailure("L-PROTO", f"{path}.{side}.arrive", "producer and consumer arrival declarations disagree"))
        for key in ("slots", "tx_bytes", "member_of"):
            if ps.get(key) != cs.get(key):
                out.append(ClauseFailure("L-PROTO", f"{path}.{side}.{key}", f"producer and consumer disagree on {key}"))
    if pp.get("init") != cp.get("init"):
        out.append(ClauseFailure("L-PROTO", f"{path}.init", "barrier ring has more than one init owner or materializer"))
    rest = lambda d: {k: v for k, v in d.items() if k not in ("full", "empty", "init")}
    if not out and rest(pp) != rest(cp):
        out.append(ClauseFailure("L-PROTO", path, "endpoint protocols differ"))
    return out


def _declared_name(decl):
    """The function a C declaration declares: the identifier in front of its parameter list."""
    if not isinstance(decl, str) or "(" not in decl:
        return None
    head = decl.split("(", 1)[0].replace("*", " ").split()
    return head[-1] if head else None


DTYPE_BITS = {"bf16": 16, "f16": 16, "fp16": 16, "f32": 32, "fp32": 32, "s32": 32, "u32": 32, "s8": 8, "u8": 8, "e4m3": 8,
              "e5m2": 8, "e4m3+ue8m0": 8}


def _tile_bytes(ep):
    tile = ep.get("tile") or {}
    n = 1
    for d in tile.get("shape", []):
        n *= d
    return n * DTYPE_BITS.get(tile.get("dtype"), 8) // 8


def _arrival_count(count, warps):
    """An arrival count is a number, or `threads(role)` / `warps(role)` of a role of the image."""
    if isinstance(count, int):
        return count
    if isinstance(count, str) and count.endswith(")") and "(" in count:
        fn, role = count[:-1].split("(", 1)
        if role in warps and fn in ("threads", "warps"):
            return warps[role] * (32 if fn == "threads" else 1)
    return None


def _role_sizes(manifests):
    sizes = {}
    for m in manifests:
        for role, r in m["stage"]["roles"].items():
            sizes[role] = r["warps"]
    return sizes


def expand_protocols(channels, manifests, cluster_size: int = 1, handles=None) -> list[dict]:
    """One expansion record per channel: barrier slot handles, arrival counts, tx bytes, depth.
    A cluster-scoped channel may collect its arrivals from the role's warps in every CTA of the
    cluster (the reference's example: pl::side{..., {"producer", 2}, 0} under .scope("cluster"),
    docs/reference/annotations.md:205-209)."""
    warps = _role_sizes(manifests)
    failures, out, inits = [], [], {}
    exports = {m["stage"]["id"]: m["stage"].get("exports", {}) for m in manifests}

    def _tx(tx, ep):
        return _tile_bytes(ep) if tx == "tile" else tx

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
                if "member_of" in s:
                    # this side completes on another channel's barrier (shared completion): the target
                    # must be a root, i.e. a side with arrivals of its own
                    target = channels.get(s["member_of"])
                    tside = (target[0][1]["protocol"].get(side) or {}) if target else {}
                    if target is None or "member_of" in tside or "arrive" not in tside:
                        failures.append(ClauseFailure("L-PROTO", f"channels.{s['member_of']}.protocol.{side}",
                                                      "member_of may only target a root barrier side"))
                    rec[side] = {"member_of": s["member_of"], "tx_bytes": _tx(s.get("tx_bytes", 0), pe)}
                    continue
                by, count = s["arrive"]["by"], _arrival_count(s["arrive"]["count"], warps)
                if by not in warps:
                    failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol.{side}.arrive.by", f"unknown role {by!r}"))
                    continue
                # one elected thread, or one lane / every thread of some of the role's warps (a role may split
                # its warps over the slots of a channel: four softmax warps per head arrive 128 strong)
                legal = {1} | {n * w for w in range(1, warps[by] + 1) for n in (1, 32)}
                if pe.get("scope") == "cluster":
                    legal |= {cluster_size * n for n in legal}
                if count not in legal:
                    failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol.{side}.arrive.count",
                                                  f"{s['arrive']['count']} arrivals cannot come from role {by!r} ({warps[by]} warps)",
                                                  {"legal": sorted(legal)}))
                tx = s.get("tx_bytes", 0)
                if isinstance(tx, dict):
                    # the root of a shared completion: its transaction count is the sum over itself and
                    # every channel whose same side names it as root
                    members = {name} | {n for n, ((_, e), _c) in channels.items()
                                        if ((e.get("protocol") or {}).get(side) or {}).get("member_of") == name}
                    if set(tx.get("sum", [])) != members or len(tx.get("sum", [])) != len(members):
                        failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol.{side}.tx_bytes.sum",
                                                      "root sum must name exactly the root and all direct members",
                                                      {"members": sorted(members)}))
                    total = sum(_tile_bytes(channels[n][0][1]) for n in members if n in channels)
                    rec[side] = {"slots": s["slots"], "count": count, "by": by, "tx_bytes": total, "sum": sorted(members)}
                else:
                    rec[side] = {"slots": s["slots"], "count": count, "by": by, "tx_bytes": _tx(tx, pe)}
            full = proto.get("full") or {}
            tx, stride = (rec.get("full") or {}).get("tx_bytes", 0), ring.get("stage_stride_bytes", 0)
            # a slot may carry padding behind its payload (alignment of the next slot), never less than it
            payload = ring.get("payload_bytes", stride)
            if (isinstance(full.get("tx_bytes", 0), int) and tx not in (0, payload, cluster_size * payload)
                    and pe["proxy"] == "async" and pe["space"] == "smem"):
                failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol.full.tx_bytes",
                                              "expected transaction bytes differ from the ring slot's payload"))
            if payload > stride:
                failures.append(ClauseFailure("L-PROTO", f"channels.{name}.ring.payload_bytes", "a slot's payload exceeds its stride"))
            init = proto.get("init", {})
            rec["init"] = init
        elif proto["kind"] == "call":
            rec["callable"] = [proto["export"], proto.get("decl", "")]
            # what the generated trampoline needs: the caller's symbol, the provider's, and the C signature
            # (an endpoint names its function as `symbol`, or spells the whole declaration as `decl`, the
            # reference's form: extern "C" __device__ float pipelink_call_scale(float);)
            cproto0 = ce.get("protocol") or {}
            caller = proto.get("symbol") or _declared_name(proto.get("decl"))
            provider = ((exports.get(cs, {}).get(cproto0.get("export")) or {}).get("symbol") or cproto0.get("symbol")
                        or _declared_name(cproto0.get("decl")))
            if caller is not None and provider is not None and proto.get("signature"):
                rec["trampoline"] = {"caller": caller, "provider": provider, "signature": proto["signature"]}
            # the provided side restates its stage's export record: declaration text and its digest
            cproto = ce.get("protocol") or {}
            record = exports.get(cs, {}).get(cproto.get("export"))
            if record is None:
                failures.append(ClauseFailure("L-SYM", f"channels.{name}.protocol.export",
                                              f"stage {cs!r} provides the channel but exports no {cproto.get('export')!r}"))
            if record is not None and "decl" in record and (
                    (cproto.get("decl"), cproto.get("decl_sha256")) != (record.get("decl"), record.get("decl_sha256"))):
                failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol",
                                              "consumer export declaration or hash disagrees with the channel"))
        elif proto["kind"] == "named_barrier":
            # pipec/src/pipec2/protocol.py:803-815: the id is a base handle of the named_barrier domain
            decl = (handles or {}).get(proto.get("id"))
            if handles is not None and (decl is None or decl.get("class") != "base" or decl.get("domain") != "named_barrier"):
                failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol",
                                              "named-barrier id handle is not declared in the named_barrier domain"))
            rec["named_barrier"] = [proto.get("id"), proto.get("count")]
        else:
            failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol.kind", f"unsupported protocol kind {proto['kind']!r}"))
        out.append(rec)
    # channels over the same physical barrier ring (the same slot handles) are initialised once: the
    # first declared states owner and materializer, a later one that differs is the failure
    declared = []
    for m in manifests:
        for ep in m.get("endpoints", []):
            if ep["name"] in channels and ep["name"] not in declared:
                declared.append(ep["name"])
    for name in declared:
        proto = channels[name][0][1].get("protocol") or {}
        ring_key = tuple((proto.get(side) or {}).get("slots") for side in ("full", "empty"))
        if proto.get("kind") != "mbarrier" or None in ring_key:
            continue
        first = inits.setdefault(ring_key, (name, proto.get("init", {})))
        if first[1] != proto.get("init", {}):
            failures.append(ClauseFailure("L-PROTO", f"channels.{name}.protocol.init",
                                          "barrier ring has more than one init owner or materializer", {"first": first[0]}))
    if failures:
        raise PipeLinkError(failures)
    return out
