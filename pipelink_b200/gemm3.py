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


class Gemm3Hosted:
    """The same GEMM opened through the host broker: the group's provider
    (stages/gemm3/host/provider.cu) is asked what it needs and writes the three parameter blocks,
    tensor maps included; this class only names the tensors. One open per set of tensors, any
    number of launches (or one captured CUDA graph) after it."""

    GROUP = Path(__file__).resolve().parent / "stages" / "gemm3" / "gemm3.host.json"

    def __init__(self, aq, asc, bq, bsc, bias, out, link_dir=None, backend=None):
        from .pipec2 import host
        link_dir = Path(link_dir or ensure_built())
        provider = link_dir.parent / "libgemm3_provider.so"
        if not provider.exists():
            from .stages.gemm3 import build
            build.build_provider(link_dir.parent)
        M, K = aq.shape
        N = bq.shape[0]
        R = host.Resource.of_tensor
        self.tensors = (aq, asc, bq, bsc, bias, out)      # keep the allocations alive
        self.session = host.open_host(
            link_dir, self.GROUP, provider, struct.pack("<IIII", M, N, K, 0),
            {"a": R(aq), "a_scales": R(asc), "b": R(bq), "b_scales": R(bsc), "bias": R(bias), "out": R(out, "write")},
            backend=backend)

    def run(self, stream=None):
        self.session.launch(stream if stream is not None else torch.cuda.current_stream().cuda_stream)

    def capture(self):
        from .pipec2 import host
        return host.CudaBackend.capture(self.session)

    def close(self):
        self.session.close()
