"""The C-ABI library loads without a GPU and exports every symbol the public headers declare."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b(plb_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "plb_moe_gemm_gate_up" in names and "plb_mxfp8_quantize" in names
    assert len(names) >= 12


def test_library_exports_every_declared_symbol(native_lib):
    for name in declared_symbols():
        assert hasattr(native_lib, name), name


def test_python_prototypes_cover_the_header(native_lib):
    from pipelink_b200 import _lib
    assert sorted(_lib.PROTOTYPES) == declared_symbols()
    assert native_lib.plb_abi_version() == 1
    assert native_lib.plb_error_string(3) == b"bad argument"


def test_argument_checks_need_no_gpu(native_lib):
    # rows not a multiple of 128 is rejected before any CUDA call
    assert native_lib.plb_mxfp8_quantize(ctypes.c_void_p(16), 100, 128, None, None, None, None, None) == 3
    assert native_lib.plb_moe_schedule_scratch_bytes(1, 2048, 8, 64) == 16 * 64 * 4


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from pipelink_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    try:
        _lib.load()
    except _lib.NativeLibraryMissing as e:
        assert "no fallback" in str(e).lower()
    else:
        raise AssertionError("load() must raise when the library is absent")
