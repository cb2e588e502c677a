"""Host for the linked three-stage MXFP8 GEMM: builds the stage parameter blocks (what the
owners' providers would write into their residue, examples/hopper-gemm-split/host/owner/provider.cpp:13-48)
and launches the linked image through ``pipec2.launcher.Session``."""
from __future__ import annotations

import ctypes
import struct
from pathlib import Path

import torch

from . import _lib
from .pipec2.launcher import Session

OUT_DIR = Path(__file__).resolve().parent / "stages" / "gemm3" / "out"


def ensure_built(depth=None) -> Path:
    link_dir = OUT_DIR / "link"
    if not (link_dir / "pipeline.cubin").exists() or not (link_dir / "one_tu.cubin").exists():
        from .stages.gemm3 import build
        build.build(OUT_DIR, depth)
    return link_dir


def tensor_map(t: torch.Tensor) -> bytes:
    rows, k = t.shape
    buf = (ctypes.c_ubyte * 128)()
    _lib.call("plb_tensor_map_2d_u8", buf, t.data_ptr(), rows, k, 128, 128, 1)
    return bytes(buf)


class Gemm3:
    """out[M, N] = bf16(silu(A_q . B_q^T + bias)); operands are MXFP8 (u8 + scale tensors)."""

    def __init__(self, link_dir=None, image="pipeline.cubin"):
        self.session = Session(link_dir or ensure_built(), image)

    def run(self, aq, asc, bq, bsc, bias, out, stream=None):
        M, K = aq.shape
        N = bq.shape[0]
        if M % 128 or N % 128 or K % 128:
            raise ValueError("M, N and K must be multiples of 128")
        s = self.session
        s.set_params("gemm.load", tensor_map(aq) + tensor_map(bq) + struct.pack("<QQii", asc.data_ptr(), bsc.data_ptr(), K, 0))
        s.set_params("gemm.mma", struct.pack("<iiii", K, 0, 0, 0))
        s.set_params("gemm.epilogue.bias-silu", struct.pack("<QQii", bias.data_ptr(), out.data_ptr(), N, 0))
        s.launch((M // 128, N // 128, 1), stream if stream is not None else torch.cuda.current_stream().cuda_stream)
        return out

    def close(self):
        self.session.close()
