"""The decode interpreter as a LINKED image: the two owners of ``stages/decode`` (the producer warp
and the sixteen interpreter warps, packed separately) joined by the link driver, launched on the
buffers of a ``DecodeSession`` in place of the library's ``plb_decode_step``.

    s = decode.DecodeSession(weights, max_seq_len=...)
    linked = LinkedDecode(s)              # or LinkedDecode(s, image="one_tu.cubin"): the single-unit control
    s.start(token, pos); linked.decode(16)

The device bodies are the library kernel's own (csrc/decode_roles.cuh), reading every shared-memory
offset and the ring depth through link-time handles, so a linked token is the library's token.
Counterpart of the reference's linked decode megakernel and its gate: the linked build within 1 % of
the single-unit build of the same sources (campaigns/megakernel/README.md).
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import torch

from . import _lib
from .pipec2.launcher import Session

OUT_DIR = Path(__file__).resolve().parent / "stages" / "decode" / "out"


def ensure_built() -> Path:
    if not all((OUT_DIR / "link" / f).exists() for f in ("pipeline.cubin", "one_tu.cubin", "link.json")):
        from .stages.decode import build
        build.build(OUT_DIR)
    return OUT_DIR / "link"


class LinkedDecode:
    def __init__(self, session, link_dir=None, image: str = "pipeline.cubin"):
        self.session = session
        self.image = Session(Path(link_dir or ensure_built()), image)
        s = session
        args = bytes(s.args)
        maps = []
        for cache in (s.k_cache, s.v_cache):
            buf = (ctypes.c_ubyte * 128)()
            _lib.call("plb_decode_kv_map", buf, cache.data_ptr(), s.layers, s.max_seq_len)
            maps.append(bytes(buf))
        self.image.set_params("decode.stream", maps[0] + maps[1] + args)
        self.image.set_params("decode.interpret", args)

    def step(self):
        """One token: the dependency counters are zeroed on the stream, then one cooperative launch."""
        s = self.session
        s.bars.zero_()
        _lib.call("plb_image_launch_cooperative", self.image._kernel, s.num_sms, self.image.link["threads"],
                  self.image.link["dyn_smem_bytes"], ctypes.addressof(self.image.params),
                  torch.cuda.current_stream().cuda_stream)

    def decode(self, steps: int, check: bool = True):
        for _ in range(steps):
            self.step()
        if check:
            self.session.status.check("after linked decode")
        return self.session.token_out

    def close(self):
        self.image.close()
