"""LTO device link through nvJitLink (ctypes), as the reference does
(pipec/src/pipec2/link.py:791-900; the library is searched for, not hard-coded)."""
from __future__ import annotations

import ctypes
import glob
import os
import shutil
import subprocess

from .model import fail

INPUT_OBJECT = 5


def nvcc() -> str:
    for cand in (os.environ.get("PLB_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    fail("P-COMPILE", "toolchain.nvcc", "nvcc not found")


def find_library() -> str:
    pats = [os.environ.get("PLB_NVJITLINK", ""), "/usr/local/cuda/lib64/libnvJitLink.so*",
            "/usr/local/cuda*/targets/x86_64-linux/lib/libnvJitLink.so*"]
    for p in pats:
        for hit in sorted(glob.glob(p)) if p else []:
            return hit
    fail("L-LINK", "toolchain.nvjitlink", "libnvJitLink not found")


def compile_lto(source: str, out: str, profile: dict, includes=(), defines=()) -> None:
    cmd = [nvcc(), "-dc", "-rdc=true", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
           "-gencode", f"arch={profile['gencode'][0]},code={profile['gencode'][1]}", "-o", out, source]
    for inc in includes:
        cmd += ["-I", str(inc)]
    for d in defines:
        cmd += [f"-D{d}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        fail("P-COMPILE", source, proc.stderr[-2000:])


def link(objects: list[tuple[str, bytes]], arch: str, extra=()) -> tuple[bytes, str]:
    """objects: (name, LTO object bytes). Returns (cubin, info log)."""
    lib = ctypes.CDLL(find_library())
    handle = ctypes.c_void_p()
    opts = [b"-lto", f"-arch={arch}".encode(), b"-O3", *[o.encode() for o in extra]]
    arr = (ctypes.c_char_p * len(opts))(*opts)

    def sym(name):
        # versioned symbols (e.g. __nvJitLinkCreate_12_9) sit behind plain-named wrappers
        return getattr(lib, name)

    def log(kind):
        n = ctypes.c_size_t()
        sym(f"nvJitLinkGet{kind}LogSize")(handle, ctypes.byref(n))
        buf = ctypes.create_string_buffer(n.value + 1)
        sym(f"nvJitLinkGet{kind}Log")(handle, buf)
        return buf.value.decode(errors="replace")

    rc = sym("nvJitLinkCreate")(ctypes.byref(handle), len(opts), arr)
    if rc != 0:
        fail("L-LINK", "nvJitLinkCreate", f"error {rc}")
    try:
        for name, data in objects:
            rc = sym("nvJitLinkAddData")(handle, INPUT_OBJECT, data, len(data), name.encode())
            if rc != 0:
                fail("L-LINK", f"nvJitLinkAddData({name})", f"error {rc}: {log('Error')}")
        rc = sym("nvJitLinkComplete")(handle)
        if rc != 0:
            fail("L-LINK", "nvJitLinkComplete", f"error {rc}: {log('Error')}")
        n = ctypes.c_size_t()
        sym("nvJitLinkGetLinkedCubinSize")(handle, ctypes.byref(n))
        cubin = ctypes.create_string_buffer(n.value)
        sym("nvJitLinkGetLinkedCubin")(handle, cubin)
        return cubin.raw, log("Info")
    finally:
        sym("nvJitLinkDestroy")(ctypes.byref(handle))
