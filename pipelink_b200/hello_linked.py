"""The hello image: ``output[i] = scale(input[i])`` with the loop and the callee in separately
packed stages (``stages/hello``), the call crossing a trampoline the link generated.

    img = HelloImage()                       # or HelloImage(image="one_tu.cubin"): the single-unit control
    img(x, out)                              # float32 CUDA tensors of one size
"""
from __future__ import annotations

import struct
from pathlib import Path

from .pipec2.launcher import Session
from .stages.hello import build as hello_build


def ensure_built() -> Path:
    out = hello_build.HERE / "out"
    if not (out / "link" / "pipeline.cubin").exists() or not (out / "link" / "one_tu.cubin").exists():
        hello_build.build(out)
    return out / "link"


class HelloImage:
    GRID = 1024     # the reference's launch of the same pair: grid 1024, block 128, no shared memory

    def __init__(self, link_dir=None, image: str = "pipeline.cubin"):
        self.session = Session(Path(link_dir or ensure_built()), image)

    def __call__(self, x, out, stream=None):
        import torch
        if x.dtype != torch.float32 or out.dtype != torch.float32 or x.numel() != out.numel() or not (x.is_cuda and out.is_cuda):
            raise ValueError("hello image: two float32 CUDA tensors of one size")
        self.session.set_params("hello.caller", struct.pack("<QQq", x.data_ptr(), out.data_ptr(), x.numel()))
        self.session.launch((self.GRID,), stream if stream is not None else torch.cuda.current_stream().cuda_stream)
        return out

    def close(self):
        self.session.close()
