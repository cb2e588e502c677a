"""The host broker against a provider with no device behind it (tests/fixtures/fake_provider.c,
compiled here with gcc against include/pipelink_host_abi_v2.h) and an in-memory backend: call
order, ownership, and every check the broker makes on what a provider answers. Failures are made
on the host, by the provider returning an error code or a wrong answer."""
import ctypes
import json
import struct
import subprocess
from pathlib import Path

import pytest

from pipelink_b200.pipec2 import host

ROOT = Path(__file__).resolve().parent.parent
MODES = {"ok": 0, "query_argument": 2, "build2_fails": 3, "build_moves_geometry": 4, "transfer_outside": 5,
         "demand_too_big": 6, "two_geometries": 8, "wrong_depth": 9, "no_geometry": 10}
GROUP = {"suffix": "fake", "args_bytes": 4, "channels": [{"id": 1, "name": "x", "rank": 1}],
         "scalars": [{"id": 1, "name": "depth", "binding": "d"}],
         "owners": [{"id": 1, "stage_id": "s.one", "channels": [1], "transfers": [{"id": 11, "channel": 1, "endpoint": "ops"}]},
                    {"id": 2, "stage_id": "s.two", "channels": [], "transfers": []}]}
LINK = {"kernel_symbol": "pipelink_kernel", "threads": 128, "dyn_smem_bytes": 1024, "cluster": [1, 1, 1],
        "params": {"total_bytes": 320, "align": 64, "entries": [["s.one", 0, 256], ["s.two", 256, 64]]},
        "bindings": {"d": [4, "solved"]},
        "protocol_expansions": [{"channel": "ops", "kind": "mbarrier", "depth": {"handle": "d"}, "stage_stride_bytes": 8192,
                                 "full": {"slots": "f", "count": 1, "by": "load", "tx_bytes": 8192}, "empty": None}]}


@pytest.fixture(scope="module")
def fake(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake")
    lib = out / "libfake_provider.so"
    subprocess.run(["gcc", "-std=c11", "-O1", "-fPIC", "-shared", "-I", str(ROOT / "include"), "-o", str(lib),
                    str(ROOT / "tests" / "fixtures" / "fake_provider.c")], check=True)
    (out / "link.json").write_text(json.dumps(LINK))
    handle = ctypes.CDLL(str(lib))
    return out, lib, handle


def _log(handle):
    buf = ctypes.create_string_buffer(1024)
    handle.fake_log(buf, 1024)
    return buf.value.decode().strip(",").split(",")


def _open(fake, mode, nbytes=1024, address=0x1000, **kw):
    out, lib, handle = fake
    handle.fake_reset()
    backend = host.MemoryBackend()
    res = {"x": host.Resource(address, nbytes, [1024], [8])}
    return backend, lambda: host.open_host(out, GROUP, lib, struct.pack("<I", MODES[mode]), res, backend=backend, **kw)


def test_records_have_the_sizes_a_c_compiler_gives_them(fake):
    """The abi report of a provider compiled from the C header equals the ctypes mirror, record by record."""
    _, _, handle = fake
    entries = (host.LayoutEntry * 64)()
    rep = host._header(host.AbiReport())
    rep.entries, rep.entry_capacity = entries, 64
    assert handle.pipelink_params_abi_fake(ctypes.byref(rep)) == 0 and rep.entry_count == len(host.ABI_TYPES)
    for i in range(rep.entry_count):
        t = host.ABI_TYPES[entries[i].abi_type_id]
        assert (entries[i].bytes, entries[i].alignment_bytes) == (ctypes.sizeof(t), ctypes.alignment(t)), t.__name__


def test_open_launch_close_order_and_ownership(fake):
    backend, opener = _open(fake, "ok")
    s = opener()
    _, _, handle = fake
    assert _log(handle) == ["abi0", "query1", "query2", "build1", "build2"]
    assert handle.fake_live(1) == 1 and handle.fake_live(2) == 1
    # each owner wrote only its own slice of the params image
    image = bytes(s.params)
    assert image[:256] == bytes([0xA1]) * 256 and image[256:320] == bytes([0xA2]) * 64
    assert s.geometry == ((3, 2, 1), (128, 1, 1), (1, 1, 1), 1024)
    assert s.transfers == [{"owner": 1, "transfer": 11, "endpoint": "ops", "ring_depth": 4, "credit_bytes_per_stage": 8192,
                            "vendor_kind": host.TRANSFER_TMA_TILED}]
    s.launch(stream=5)
    s.launch(stream=5)
    assert len(backend.launches) == 2 and backend.launches[0][0] == s.geometry and backend.launches[0][2] == 5
    assert _log(handle)[-1] == "build2", "launch makes no provider call"
    s.close()
    s.close()      # idempotent: every session is released exactly once, in reverse build order
    assert _log(handle)[5:] == ["release2", "release1"] and handle.fake_live(1) == 0 and handle.fake_live(2) == 0
    assert len(backend.freed) == 1, "the workspace the broker allocated is freed"
    with pytest.raises(host.HostError):
        s.launch()


@pytest.mark.parametrize("mode,clause,code,path", [
    ("query_argument", "L-HOSTCALL", 3, "owners.1.query"),
    ("demand_too_big", "L-HOSTCHAN", 0, "channels.x.bytes"),
    ("two_geometries", "L-HOSTGEOM", 0, "owners.2.geometry"),
    ("no_geometry", "L-HOSTGEOM", 0, "groups.fake"),
    ("build2_fails", "L-HOSTCALL", 6, "owners.2.build"),
    ("build_moves_geometry", "L-HOSTGEOM", 0, "owners.1.build"),
    ("transfer_outside", "L-HOSTCHAN", 0, "owners.1.transfers.11"),
    ("wrong_depth", "L-HOSTCHAN", 0, "owners.1.transfers.11.ring_depth"),
])
def test_provider_misbehaviour_is_reported_and_nothing_leaks(fake, mode, clause, code, path):
    backend, opener = _open(fake, mode)
    with pytest.raises(host.HostError) as e:
        opener()
    assert (e.value.clause, e.value.code) == (clause, code) and e.value.path.startswith(path), str(e.value)
    _, _, handle = fake
    assert handle.fake_live(1) == 0 and handle.fake_live(2) == 0, "sessions built before the failure are released"
    log = _log(handle)
    builds, releases = [x for x in log if x.startswith("build")], [x for x in log if x.startswith("release")]
    built_ok = [b for b in builds if not (mode == "build2_fails" and b == "build2")]
    assert releases == [b.replace("build", "release") for b in reversed(built_ok)]
    assert backend.launches == []


def test_caller_side_checks(fake):
    _, opener = _open(fake, "ok", address=0x1008)      # misaligned for the owner's 16-byte demand
    with pytest.raises(host.HostError) as e:
        opener()
    assert e.value.clause == "L-HOSTCHAN" and e.value.path == "channels.x.alignment"
    out, lib, _ = fake
    with pytest.raises(host.HostError) as e:
        host.open_host(out, GROUP, lib, b"\0" * 4, {}, backend=host.MemoryBackend())
    assert e.value.path == "channels.x"
    with pytest.raises(host.HostError) as e:
        host.open_host(out, GROUP, lib, b"\0" * 8, {"x": host.Resource(0x1000, 1024, [1024], [8])}, backend=host.MemoryBackend())
    assert e.value.path == "groups.fake.args"
    with pytest.raises(host.HostError) as e:
        host.open_host(out, dict(GROUP, suffix="absent"), lib, b"\0" * 4, {"x": host.Resource(0x1000, 1024, [1024], [8])},
                       backend=host.MemoryBackend())
    assert e.value.clause == "L-HOSTABI"


def test_abi_mismatch_and_failing_release(fake, monkeypatch):
    backend, opener = _open(fake, "ok")
    monkeypatch.setenv("FAKE_PROVIDER_ABI_SIZE", "1")
    with pytest.raises(host.HostError) as e:
        opener()
    assert e.value.clause == "L-HOSTABI" and "Common" in str(e.value)
    monkeypatch.delenv("FAKE_PROVIDER_ABI_SIZE")
    backend, opener = _open(fake, "ok")
    s = opener()
    monkeypatch.setenv("FAKE_PROVIDER_RELEASE1_FAILS", "1")
    with pytest.raises(host.HostError) as e:
        s.close()
    assert (e.value.clause, e.value.code) == ("L-HOSTCALL", 7)
    _, _, handle = fake
    assert _log(handle)[-2:] == ["release2", "release1"], "a failing release does not stop the others"


def test_gemm3_provider_answers_query_without_a_device(tmp_path):
    """The real provider of the three-stage GEMM: report and query need no GPU; build needs the
    driver's tensor-map encoder, so without one it must fail cleanly with PLK_E_BUILD."""
    from pipelink_b200.stages.gemm3 import build as g3
    lib = g3.build_provider(tmp_path)
    handle = ctypes.CDLL(str(lib))
    for verb in ("abi", "query", "build", "release"):
        assert hasattr(handle, f"pipelink_params_{verb}_gemm3")
    link = {"kernel_symbol": "pipelink_kernel", "threads": 192, "dyn_smem_bytes": 202992, "cluster": [1, 1, 1],
            "params": {"total_bytes": 384, "align": 64, "entries": [["gemm.load", 0, 320], ["gemm.mma", 320, 16], ["gemm.epilogue.bias-silu", 336, 32]]},
            "bindings": {"pipelink_gemm_depth": [6, "solved"]},
            "protocol_expansions": [{"channel": "operands", "kind": "mbarrier", "depth": {"handle": "pipelink_gemm_depth"},
                                     "stage_stride_bytes": g3.SLOT, "full": {"tx_bytes": g3.SLOT}, "empty": None}]}
    (tmp_path / "link.json").write_text(json.dumps(link))
    M, N, K = 256, 384, 512
    R = host.Resource
    res = {"a": R(0x10000, M * K, [M, K], [K * 8, 8]), "a_scales": R(0x200000, M * K // 32, [M // 128, K // 128, 32, 16], [K // 128 * 4096, 4096, 128, 8]),
           "b": R(0x300000, N * K, [N, K], [K * 8, 8]), "b_scales": R(0x400000, N * K // 32, [N // 128, K // 128, 32, 16], [K // 128 * 4096, 4096, 128, 8]),
           "bias": R(0x500000, N * 2, [N], [16]), "out": R(0x600000, M * N * 2, [M, N], [N * 16, 16], access="write")}
    group = ROOT / "pipelink_b200" / "stages" / "gemm3" / "gemm3.host.json"
    backend = host.MemoryBackend()
    try:
        s = host.open_host(tmp_path, group, lib, struct.pack("<IIII", M, N, K, 0), res, backend=backend)
    except host.HostError as e:
        assert (e.clause, e.code, e.path) == ("L-HOSTCALL", 6, "owners.1.build"), str(e)
    else:   # a machine with a driver: the whole open succeeds
        assert s.geometry[0] == (M // 128, N // 128, 1) and [t["ring_depth"] for t in s.transfers] == [6, 6]
        s.close()
    small = dict(res, a=R(0x10000, M * K - 1, [M, K], [K * 8, 8]))
    with pytest.raises(host.HostError) as e:
        host.open_host(tmp_path, group, lib, struct.pack("<IIII", M, N, K, 0), small, backend=backend)
    assert e.value.path == "channels.a.bytes"
    with pytest.raises(host.HostError) as e:
        host.open_host(tmp_path, group, lib, struct.pack("<IIII", M, N, 100, 0), res, backend=backend)
    assert (e.value.clause, e.value.code) == ("L-HOSTCALL", 3)
