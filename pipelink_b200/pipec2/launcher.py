"""Launch a linked image: the host-less session of the reference
(pipec/src/pipec2/launcher.py:171-189 ``open_hostless`` / ``launch`` / ``time(n)``)."""
from __future__ import annotations

import ctypes
import json
from pathlib import Path

from .. import _lib


class Session:
    def __init__(self, link_dir, image: str = "pipeline.cubin"):
        link_dir = Path(link_dir)
        self.link = json.loads((link_dir / "link.json").read_text())
        self.image = (link_dir / image).read_bytes()
        self._lib_handle, self._kernel = ctypes.c_void_p(), ctypes.c_void_p()
        _lib.call("plb_image_load", self.image, self.link["kernel_symbol"].encode(), self.link["dyn_smem_bytes"],
                  ctypes.byref(self._lib_handle), ctypes.byref(self._kernel))
        self.params = (ctypes.c_ubyte * self.link["params"]["total_bytes"])()
        self.offsets = {e[0]: (e[1], e[2]) for e in self.link["params"]["entries"]}

    def set_params(self, stage_id: str, blob: bytes):
        off, size = self.offsets[stage_id]
        if len(blob) > size:
            raise ValueError(f"{stage_id}: {len(blob)} bytes exceed the {size}-byte parameter block")
        ctypes.memmove(ctypes.addressof(self.params) + off, blob, len(blob))

    def launch(self, grid, stream=None):
        gx, gy, gz = (tuple(grid) + (1, 1))[:3]
        _lib.call("plb_image_launch", self._kernel, gx, gy, gz, self.link["threads"], self.link["dyn_smem_bytes"],
                  ctypes.addressof(self.params), stream)

    def time(self, grid, n: int = 20, stream=None) -> float:
        import torch
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.launch(grid, stream)
        torch.cuda.synchronize()
        a.record()
        for _ in range(n):
            self.launch(grid, torch.cuda.current_stream().cuda_stream)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    def close(self):
        if self._lib_handle:
            _lib.call("plb_image_unload", self._lib_handle)
            self._lib_handle = ctypes.c_void_p()
