"""Host broker: opens a linked image together with its params providers.

The hosted counterpart of ``launcher.Session`` and the stand-in for the reference's broker
(pipec/src/pipec2/host/broker.py: ``open_host`` -> ``HostSession.launch`` / ``close``;
pipec/src/pipec2/host/cuda.py: ``CudaBackend.launch`` / ``capture``). The caller names the
tensors; every owner of a params group is asked what it needs (``query``), handed the device
addresses (``build``) and writes its own parameter block, tensor maps included, into its slice
of the params image. Call order on the opening thread, as in the reference
(broker.py:847): abi report -> query (all owners) -> build (all owners); ``launch`` makes no
provider call; ``close`` releases the sessions in reverse build order, each exactly once.

What the broker checks, with the clause it reports (``HostError.clause``):
  L-HOSTABI    the provider's record sizes / alignments equal this process's (abi report)
  L-HOSTCALL   a provider call returned PLK_E_* (``HostError.code``)
  L-HOSTCHAN   demands fit the caller's tensors (bytes, alignment, rank, access); transfer
               reports stay inside the residue and agree with the linked endpoint
               (ring depth, stage stride, bytes per stage)
  L-HOSTGEOM   exactly one owner states the launch geometry, it fits the link, and no build
               changes it
Group description (``*.host.json`` beside the stage sources): suffix, args size, owners
{id, stage_id, channels, transfers[{id, channel, endpoint}]}, channels {id, name, rank},
scalars {id, name}.
"""
from __future__ import annotations

import ctypes
import json
from ctypes import POINTER, Structure, c_int64, c_size_t, c_uint8, c_uint32, c_uint64, c_void_p
from pathlib import Path

ABI_VERSION = 2
PLK_CODES = {0: "PLK_OK", 1: "PLK_E_VERSION", 2: "PLK_E_CAPACITY", 3: "PLK_E_ARGUMENT", 4: "PLK_E_CONTRACT",
             5: "PLK_E_RESOURCE", 6: "PLK_E_BUILD", 7: "PLK_E_RELEASE"}
ACCESS = {"read": 1, "write": 2, "read_write": 3}
TRANSFER_TMA_TILED = 1
MAX_RANK = 5


class HostError(Exception):
    def __init__(self, clause: str, path: str, message: str, code: int = 0):
        super().__init__(f"[{clause}] {path}: {message}" + (f" ({PLK_CODES.get(code, code)})" if code else ""))
        self.clause, self.path, self.code = clause, path, code


# ---- records of include/pipelink_host_abi_v2.h, same field order ------------------------------
class Header(Structure):
    _fields_ = [("abi_version", c_uint32), ("struct_bytes", c_uint32)]


class Digest(Structure):
    _fields_ = [("sha256", c_uint8 * 32)]


class ProfileDigest(Structure):
    _fields_ = [("dtypes", Digest)]


class Dim3(Structure):
    _fields_ = [("x", c_uint32), ("y", c_uint32), ("z", c_uint32)]


class Scalar(Structure):
    _fields_ = [("scalar_id", c_uint32), ("scalar_type", c_uint32), ("value_bits", c_uint64)]


class SharedScalars(Structure):
    _fields_ = [("header", Header), ("image_bytes", c_uint64), ("record_count", c_uint32), ("record_offset", c_uint32)]


class TensorMeta(Structure):
    _fields_ = [("channel_id", c_uint32), ("dtype_id", c_uint32), ("rank", c_uint32), ("access", c_uint32),
                ("allocation_bytes", c_uint64), ("alignment_bytes", c_uint64), ("origin_byte_offset", c_uint64),
                ("origin_bit_offset", c_uint32), ("reserved", c_uint32), ("extents", POINTER(c_uint64)),
                ("bit_strides", POINTER(c_int64))]


class Geometry(Structure):
    _fields_ = [("geometry_present", c_uint32), ("launch_required", c_uint32), ("grid", Dim3), ("block", Dim3),
                ("cluster", Dim3), ("reserved", c_uint32), ("dynamic_smem_bytes", c_uint64)]

    def key(self):
        d = lambda v: (v.x, v.y, v.z)
        return (self.geometry_present, self.launch_required, d(self.grid), d(self.block), d(self.cluster), self.dynamic_smem_bytes)


class Domain(Structure):
    _fields_ = [("domain_id", c_uint32), ("rank", c_uint32), ("world", c_uint32), ("reserved", c_uint32)]


class Common(Structure):
    _fields_ = [("header", Header), ("owner_id", c_uint32), ("channel_count", c_uint32), ("domain_count", c_uint32),
                ("reserved", c_uint32), ("shared", POINTER(SharedScalars)), ("channels", POINTER(TensorMeta)),
                ("domains", POINTER(Domain)), ("block", Dim3), ("cluster", Dim3), ("dynamic_smem_bytes", c_uint64),
                ("profile", ProfileDigest), ("owner_contract", Digest)]


class ChannelDemand(Structure):
    _fields_ = [("channel_id", c_uint32), ("dtype_id", c_uint32), ("rank", c_uint32), ("access", c_uint32),
                ("minimum_allocation_bytes", c_uint64), ("alignment_bytes", c_uint64), ("extents", POINTER(c_uint64)),
                ("bit_strides", POINTER(c_int64))]


class WorkspaceDemand(Structure):
    _fields_ = [("workspace_id", c_uint32), ("reserved", c_uint32), ("bytes", c_uint64), ("alignment_bytes", c_uint64)]


class Demands(Structure):
    _fields_ = [("header", Header), ("channel_count", c_uint32), ("channel_capacity", c_uint32),
                ("channels", POINTER(ChannelDemand)), ("workspace_count", c_uint32), ("workspace_capacity", c_uint32),
                ("workspaces", POINTER(WorkspaceDemand)), ("geometry", Geometry)]


class DeviceResource(Structure):
    _fields_ = [("channel_id", c_uint32), ("access", c_uint32), ("allocation_address", c_uint64),
                ("allocation_bytes", c_uint64), ("origin_byte_offset", c_uint64), ("origin_bit_offset", c_uint32),
                ("domain_id", c_uint32), ("peer_addresses", POINTER(c_uint64)), ("multicast_address", c_uint64)]


class WorkspaceResource(Structure):
    _fields_ = [("workspace_id", c_uint32), ("reserved", c_uint32), ("device_address", c_uint64), ("bytes", c_uint64),
                ("alignment_bytes", c_uint64)]


class Resources(Structure):
    _fields_ = [("header", Header), ("channel_count", c_uint32), ("workspace_count", c_uint32),
                ("channels", POINTER(DeviceResource)), ("workspaces", POINTER(WorkspaceResource)),
                ("shared", POINTER(SharedScalars)), ("cuda_stream_token", c_uint64), ("geometry", Geometry)]


class TmaTiledDetail(Structure):
    _fields_ = [("swizzle", c_uint32), ("rank", c_uint32), ("box_elements", c_uint64 * 5), ("element_strides", c_uint32 * 5),
                ("reserved", c_uint32)]


class TransferReport(Structure):
    _fields_ = [("transfer_id", c_uint32), ("access", c_uint32), ("residue_offset", c_uint64),
                ("representation_bytes", c_uint64), ("representation_align", c_uint64), ("storage_dtype_id", c_uint32),
                ("ring_depth", c_uint32), ("ring_stage_stride_bytes", c_uint64), ("footprint_bytes_per_stage", c_uint64),
                ("credit_bytes_per_stage", c_uint64), ("source_origin_bits", c_uint64), ("source_span_bits", c_uint64),
                ("vendor_kind", c_uint32), ("reserved", c_uint32), ("vendor_detail", c_void_p)]


class LayoutEntry(Structure):
    _fields_ = [("abi_type_id", c_uint32), ("reserved", c_uint32), ("bytes", c_uint64), ("alignment_bytes", c_uint64),
                ("compiler_layout", Digest)]


class AbiReport(Structure):
    _fields_ = [("header", Header), ("entry_count", c_uint32), ("entry_capacity", c_uint32), ("entries", POINTER(LayoutEntry)),
                ("profile", ProfileDigest), ("owner_contract", Digest)]


ABI_TYPES = {0x70000001: AbiReport, 0x70000002: ChannelDemand, 0x70000003: Common, 0x70000004: Demands,
             0x70000005: TmaTiledDetail, 0x70000006: DeviceResource, 0x70000007: Digest, 0x70000008: Dim3,
             0x70000009: Geometry, 0x7000000A: Header, 0x7000000B: LayoutEntry, 0x7000000C: ProfileDigest,
             0x7000000D: Resources, 0x7000000E: Scalar, 0x7000000F: SharedScalars, 0x70000010: TransferReport,
             0x70000011: TensorMeta, 0x70000012: WorkspaceDemand, 0x70000013: WorkspaceResource, 0x70000014: Domain}


def _header(rec):
    rec.header = Header(ABI_VERSION, ctypes.sizeof(type(rec)))
    return rec


# ---- caller-side facts -------------------------------------------------------------------------
class Resource:
    """One caller tensor: device address of its allocation, bytes, and how it is shaped."""

    def __init__(self, address: int, nbytes: int, extents, bit_strides, *, access="read", alignment=256, origin_byte_offset=0):
        self.address, self.nbytes = int(address), int(nbytes)
        self.extents, self.bit_strides = tuple(int(e) for e in extents), tuple(int(s) for s in bit_strides)
        self.access, self.alignment, self.origin_byte_offset = ACCESS[access], int(alignment), int(origin_byte_offset)

    @classmethod
    def of_tensor(cls, t, access="read"):
        bits = t.element_size() * 8
        return cls(t.data_ptr(), t.numel() * t.element_size(), t.shape, [s * bits for s in t.stride()], access=access,
                   alignment=256 if t.data_ptr() % 256 == 0 else 16)


class MemoryBackend:
    """No device: hands out fake addresses and records launches. For tests of the broker's own
    logic (the reference tests its broker the same way, pipec/tests/test_host_broker.py)."""

    def __init__(self):
        self.launches, self.next_address, self.freed = [], 0x7F0000000000, []

    def allocate(self, nbytes: int, alignment: int):
        a = (self.next_address + alignment - 1) // alignment * alignment
        self.next_address = a + nbytes
        return a, ("mem", a)

    def free(self, token):
        self.freed.append(token)

    def load(self, link_dir, link):
        return None

    def launch(self, kernel, geometry, params, stream):
        self.launches.append((geometry, bytes(params), stream))

    def unload(self, kernel):
        pass


class CudaBackend:
    """Launches through the library's image entry points; workspaces are torch allocations."""

    def allocate(self, nbytes: int, alignment: int):
        import torch
        buf = torch.empty(nbytes + alignment, dtype=torch.uint8, device="cuda")
        a = (buf.data_ptr() + alignment - 1) // alignment * alignment
        return a, buf

    def free(self, token):
        del token

    def load(self, link_dir, link):
        from .. import _lib
        image = (Path(link_dir) / "pipeline.cubin").read_bytes()
        lib, kernel = c_void_p(), c_void_p()
        _lib.call("plb_image_load", image, link["kernel_symbol"].encode(), link["dyn_smem_bytes"], ctypes.byref(lib), ctypes.byref(kernel))
        return (lib, kernel)

    def launch(self, kernel, geometry, params, stream):
        from .. import _lib
        grid, block, _, smem = geometry
        _lib.call("plb_image_launch", kernel[1], grid[0], grid[1], grid[2], block[0], smem, ctypes.addressof(params), stream)

    def unload(self, kernel):
        from .. import _lib
        _lib.call("plb_image_unload", kernel[0])

    @staticmethod
    def capture(session, stream=None):
        """Records one launch of `session` into a CUDA graph and returns it (replay with .replay())."""
        import torch
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            session.launch(side.cuda_stream)            # warm-up outside capture: module load, first-use set-up
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                session.launch(side.cuda_stream)
        torch.cuda.current_stream().wait_stream(side)
        return graph


class _Owner:
    def __init__(self, spec, fns):
        self.spec, self.fns = spec, fns
        self.session = c_void_p()
        self.keep = []          # ctypes storage that must outlive the provider's session


class HostSession:
    def __init__(self, backend, kernel, geometry, params, owners, workspaces, link):
        self.backend, self.kernel, self.geometry, self.params = backend, kernel, geometry, params
        self.owners, self.workspaces, self.link = owners, workspaces, link
        self.transfers = []
        self.closed = False

    def launch(self, stream: int | None = None):
        if self.closed:
            raise HostError("L-HOSTCALL", "session", "launch after close")
        self.backend.launch(self.kernel, self.geometry, self.params, stream)

    def close(self):
        """Releases every built owner in reverse build order, each exactly once; a failing release
        does not stop the others and is reported after all of them ran."""
        if self.closed:
            return
        self.closed = True
        errors = []
        for owner in reversed(self.owners):
            if owner.session:
                rc = owner.fns["release"](owner.session)
                owner.session = c_void_p()
                if rc != 0:
                    errors.append(HostError("L-HOSTCALL", f"owners.{owner.spec['id']}.release", "provider release failed", rc))
        for token in self.workspaces:
            self.backend.free(token)
        if self.kernel is not None:
            self.backend.unload(self.kernel)
        if errors:
            raise errors[0]

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()


def _load_provider(path, suffix):
    lib = ctypes.CDLL(str(path))
    fns = {}
    for verb in ("abi", "query", "build", "release"):
        name = f"pipelink_params_{verb}_{suffix}"
        try:
            fns[verb] = getattr(lib, name)
        except AttributeError as e:
            raise HostError("L-HOSTABI", f"providers.{suffix}", f"provider does not export {name}") from e
        fns[verb].restype = ctypes.c_int
    fns["abi"].argtypes = [POINTER(AbiReport)]
    fns["query"].argtypes = [POINTER(Common), c_void_p, POINTER(Demands)]
    fns["build"].argtypes = [POINTER(Common), c_void_p, POINTER(Resources), c_void_p, c_size_t, POINTER(TransferReport),
                             c_uint32, POINTER(c_void_p)]
    fns["release"].argtypes = [c_void_p]
    return lib, fns


def _check_abi(fns, suffix):
    entries = (LayoutEntry * 64)()
    report = _header(AbiReport())
    report.entries, report.entry_capacity = entries, 64
    rc = fns["abi"](ctypes.byref(report))
    if rc != 0:
        raise HostError("L-HOSTCALL", f"providers.{suffix}.abi", "provider abi report failed", rc)
    seen = {}
    for i in range(report.entry_count):
        e = entries[i]
        seen[e.abi_type_id] = (e.bytes, e.alignment_bytes)
    for type_id, struct in ABI_TYPES.items():
        mine = (ctypes.sizeof(struct), ctypes.alignment(struct))
        if seen.get(type_id) != mine:
            raise HostError("L-HOSTABI", f"providers.{suffix}.abi", f"record 0x{type_id:08x} ({struct.__name__}) is "
                            f"{seen.get(type_id)} in the provider and {mine} here")


def _scalar_image(scalars: dict[int, int]):
    n = len(scalars)
    size = ctypes.sizeof(SharedScalars) + n * ctypes.sizeof(Scalar)
    buf = (c_uint8 * size)()
    head = SharedScalars.from_buffer(buf)
    head.header = Header(ABI_VERSION, ctypes.sizeof(SharedScalars))
    head.image_bytes, head.record_count, head.record_offset = size, n, ctypes.sizeof(SharedScalars)
    recs = (Scalar * n).from_buffer(buf, ctypes.sizeof(SharedScalars)) if n else None
    for i, (sid, value) in enumerate(sorted(scalars.items())):
        recs[i] = Scalar(sid, 1, int(value))
    return buf, ctypes.cast(buf, POINTER(SharedScalars))


def open_host(link_dir, group, provider_path, args: bytes, resources: dict, *, scalars=None, backend=None, stream_token=0):
    """link_dir: a linked pipeline (link.json, pipeline.cubin). group: the params group description
    (dict or path to ``*.host.json``). resources: channel name -> Resource. Returns a HostSession."""
    link_dir = Path(link_dir)
    link = json.loads((link_dir / "link.json").read_text())
    if not isinstance(group, dict):
        group = json.loads(Path(group).read_text())
    backend = backend or CudaBackend()
    suffix = group["suffix"]
    if len(args) != group["args_bytes"]:
        raise HostError("L-HOSTCALL", f"groups.{suffix}.args", f"args are {len(args)} bytes, the group declares {group['args_bytes']}")
    lib, fns = _load_provider(provider_path, suffix)
    _check_abi(fns, suffix)

    channels = {c["id"]: c for c in group["channels"]}
    for c in channels.values():
        if c["name"] not in resources:
            raise HostError("L-HOSTCHAN", f"channels.{c['name']}", "the caller supplied no resource for this channel")
        if len(resources[c["name"]].extents) != c["rank"]:
            raise HostError("L-HOSTCHAN", f"channels.{c['name']}.rank", f"resource rank {len(resources[c['name']].extents)} differs from the declared rank {c['rank']}")
    bindings = {k: v[0] for k, v in link["bindings"].items()}
    scalar_values = {s["id"]: (scalars or {}).get(s["name"], bindings.get(s.get("binding", ""), 0)) for s in group.get("scalars", [])}
    scalar_buf, shared = _scalar_image(scalar_values)
    offsets = {e[0]: (e[1], e[2]) for e in link["params"]["entries"]}
    params = (c_uint8 * max(link["params"]["total_bytes"], 1))()
    block, cluster = (link["threads"], 1, 1), tuple(link.get("cluster", (1, 1, 1)))
    args_buf = ctypes.create_string_buffer(args, len(args))
    owners = [_Owner(spec, fns) for spec in sorted(group["owners"], key=lambda o: o["id"])]
    keep = [lib, scalar_buf, args_buf]

    def common_for(owner):
        ids = owner.spec["channels"]
        metas = (TensorMeta * max(len(ids), 1))()
        for i, cid in enumerate(ids):
            r = resources[channels[cid]["name"]]
            ext, strides = (c_uint64 * MAX_RANK)(*r.extents), (c_int64 * MAX_RANK)(*r.bit_strides)
            owner.keep += [ext, strides]
            metas[i] = TensorMeta(cid, 0, len(r.extents), r.access, r.nbytes, r.alignment, r.origin_byte_offset, 0, 0,
                                  ctypes.cast(ext, POINTER(c_uint64)), ctypes.cast(strides, POINTER(c_int64)))
        c = _header(Common())
        c.owner_id, c.channel_count, c.domain_count = owner.spec["id"], len(ids), 0
        c.shared, c.channels = shared, metas
        c.block, c.cluster, c.dynamic_smem_bytes = Dim3(*block), Dim3(*cluster), link["dyn_smem_bytes"]
        owner.keep += [metas, c]
        return c

    # ---- query every owner
    geometry, workspace_demands = None, []
    for owner in owners:
        owner.common = common_for(owner)
        ids = owner.spec["channels"]
        dem_ch = (ChannelDemand * max(len(ids), 1))()
        for i, cid in enumerate(ids):
            ext, strides = (c_uint64 * MAX_RANK)(), (c_int64 * MAX_RANK)()
            owner.keep += [ext, strides]
            dem_ch[i] = ChannelDemand(cid, 0, channels[cid]["rank"], 0, 0, 0, ctypes.cast(ext, POINTER(c_uint64)),
                                      ctypes.cast(strides, POINTER(c_int64)))
        dem_ws = (WorkspaceDemand * 8)()
        dem = _header(Demands())
        dem.channels, dem.channel_capacity, dem.workspaces, dem.workspace_capacity = dem_ch, len(ids), dem_ws, 8
        rc = fns["query"](ctypes.byref(owner.common), args_buf, ctypes.byref(dem))
        if rc != 0:
            raise HostError("L-HOSTCALL", f"owners.{owner.spec['id']}.query", "provider query failed", rc)
        if dem.channel_count > len(ids) or dem.workspace_count > 8:
            raise HostError("L-HOSTCHAN", f"owners.{owner.spec['id']}.query", "provider reported more demands than the capacity it was given")
        for i in range(dem.channel_count):
            d = dem_ch[i]
            if d.channel_id not in ids:
                raise HostError("L-HOSTCHAN", f"owners.{owner.spec['id']}.channels", f"demand for undeclared channel {d.channel_id}")
            name = channels[d.channel_id]["name"]
            r = resources[name]
            if r.nbytes - r.origin_byte_offset < d.minimum_allocation_bytes:
                raise HostError("L-HOSTCHAN", f"channels.{name}.bytes", f"owner needs {d.minimum_allocation_bytes} bytes, the resource has {r.nbytes - r.origin_byte_offset}")
            if d.alignment_bytes and (r.address + r.origin_byte_offset) % d.alignment_bytes:
                raise HostError("L-HOSTCHAN", f"channels.{name}.alignment", f"owner needs {d.alignment_bytes}-byte alignment")
            if d.access & ~r.access:
                raise HostError("L-HOSTCHAN", f"channels.{name}.access", "owner needs an access the caller did not grant")
            want = tuple(d.extents[k] for k in range(d.rank))
            if want != r.extents:
                raise HostError("L-HOSTCHAN", f"channels.{name}.extents", f"owner expects extents {want}, the resource has {r.extents}")
        for i in range(dem.workspace_count):
            workspace_demands.append((owner, dem_ws[i].workspace_id, dem_ws[i].bytes, max(dem_ws[i].alignment_bytes, 16)))
        if dem.geometry.geometry_present:
            if geometry is not None:
                raise HostError("L-HOSTGEOM", f"owners.{owner.spec['id']}.geometry", "more than one owner states the launch geometry")
            geometry = Geometry.from_buffer_copy(dem.geometry)
        owner.keep += [dem_ch, dem_ws, dem]
    if geometry is None:
        raise HostError("L-HOSTGEOM", f"groups.{suffix}", "no owner states the launch geometry")
    if (geometry.block.x, geometry.block.y, geometry.block.z) != block or geometry.dynamic_smem_bytes != link["dyn_smem_bytes"]:
        raise HostError("L-HOSTGEOM", f"groups.{suffix}.geometry", "block or shared-memory size differs from the linked image")
    if 0 in (geometry.grid.x, geometry.grid.y, geometry.grid.z):
        raise HostError("L-HOSTGEOM", f"groups.{suffix}.geometry.grid", "empty grid")

    # ---- workspaces, then build every owner; a failure releases what was built, in reverse
    tokens, ws_by_owner = [], {}
    for owner, wid, nbytes, align in workspace_demands:
        address, token = backend.allocate(nbytes, align)
        tokens.append(token)
        ws_by_owner.setdefault(id(owner), []).append(WorkspaceResource(wid, 0, address, nbytes, align))
    session = HostSession(backend, None, None, params, [], tokens, link)
    try:
        for owner in owners:
            ids = owner.spec["channels"]
            dev = (DeviceResource * max(len(ids), 1))()
            for i, cid in enumerate(ids):
                r = resources[channels[cid]["name"]]
                dev[i] = DeviceResource(cid, r.access, r.address, r.nbytes, r.origin_byte_offset, 0, 0, None, 0)
            ws_list = ws_by_owner.get(id(owner), [])
            ws = (WorkspaceResource * max(len(ws_list), 1))(*ws_list)
            res = _header(Resources())
            res.channel_count, res.workspace_count, res.channels, res.workspaces = len(ids), len(ws_list), dev, ws
            res.shared, res.cuda_stream_token, res.geometry = shared, stream_token, geometry
            decl = owner.spec.get("transfers", [])
            reports = (TransferReport * max(len(decl), 1))()
            for i, t in enumerate(decl):
                reports[i].transfer_id = t["id"]
            off, size = offsets[owner.spec["stage_id"]]
            before = geometry.key()
            rc = fns["build"](ctypes.byref(owner.common), args_buf, ctypes.byref(res), ctypes.addressof(params) + off, size,
                              reports, len(decl), ctypes.byref(owner.session))
            owner.keep += [dev, ws, res, reports]
            if rc != 0:
                owner.session = c_void_p()
                raise HostError("L-HOSTCALL", f"owners.{owner.spec['id']}.build", "provider build failed", rc)
            session.owners.append(owner)
            if res.geometry.key() != before:
                raise HostError("L-HOSTGEOM", f"owners.{owner.spec['id']}.build", "build changed the launch geometry")
            for i, t in enumerate(decl):
                session.transfers.append(_check_transfer(owner, t, reports[i], size, link))
        session.geometry = ((geometry.grid.x, geometry.grid.y, geometry.grid.z), block, cluster, link["dyn_smem_bytes"])
        session.kernel = backend.load(link_dir, link)
    except Exception:
        try:
            session.close()
        finally:
            pass
        raise
    session.keep = keep
    return session


def _check_transfer(owner, decl, rep, residue_bytes, link):
    path = f"owners.{owner.spec['id']}.transfers.{decl['id']}"
    if rep.transfer_id != decl["id"]:
        raise HostError("L-HOSTCHAN", path, "provider overwrote the transfer id")
    if rep.residue_offset + rep.representation_bytes > residue_bytes:
        raise HostError("L-HOSTCHAN", path, "representation lies outside the owner's residue")
    if rep.representation_align and rep.residue_offset % rep.representation_align:
        raise HostError("L-HOSTCHAN", path, "representation is misaligned inside the residue")
    exp = next((e for e in link["protocol_expansions"] if e["channel"] == decl["endpoint"]), None)
    if exp is None:
        raise HostError("L-HOSTCHAN", path, f"the linked image has no channel {decl['endpoint']!r}")
    depth = exp["depth"]
    depth = link["bindings"][depth["handle"]][0] if isinstance(depth, dict) and "handle" in depth else (depth or {}).get("fixed", 1)
    if rep.ring_depth != depth:
        raise HostError("L-HOSTCHAN", path + ".ring_depth", f"owner addresses a ring of {rep.ring_depth}, the link solved {depth}")
    if rep.ring_stage_stride_bytes != exp["stage_stride_bytes"]:
        raise HostError("L-HOSTCHAN", path + ".ring_stage_stride_bytes", "stage stride differs from the linked endpoint")
    tx = (exp.get("full") or {}).get("tx_bytes", 0)
    if rep.vendor_kind == TRANSFER_TMA_TILED:
        if rep.representation_bytes != 128 or rep.vendor_detail is None:
            raise HostError("L-HOSTCHAN", path, "a tiled tensor map is 128 bytes and carries its detail record")
        if rep.credit_bytes_per_stage > tx or rep.footprint_bytes_per_stage > exp["stage_stride_bytes"]:
            raise HostError("L-HOSTCHAN", path, "bytes per stage exceed what the endpoint's barrier expects")
    return {"owner": owner.spec["id"], "transfer": decl["id"], "endpoint": decl["endpoint"], "ring_depth": rep.ring_depth,
            "credit_bytes_per_stage": rep.credit_bytes_per_stage, "vendor_kind": rep.vendor_kind}
