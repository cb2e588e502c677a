"""Causal prefill attention as LINKED images: the owners of ``stages/attention`` (load, MMA, gather
and softmax, packed separately, two forms each of load / gather / softmax) joined by the link
driver into compositions, launched here in place of the library's ``plb_attention_fwd``.

    linked = LinkedAttention()                       # loads the images
    out, lse = linked.forward(q, k, v, window=0, softcap=0.0)

The device bodies are the library kernel's own (csrc/attention_roles.cuh), reading barrier slots,
tile offsets, tensor-memory columns and the K/V ring depth through link-time handles, so a linked
launch computes the library launch's bits. Which softmax owner an image holds decides whether the
soft cap applies: a link-time variant, as in the reference's attention family
(campaigns/attention/src/sm90/stage_score_softcap.cu).
"""
from __future__ import annotations

import ctypes
import math
import struct
from pathlib import Path

import numpy as np
import torch

from . import _lib, attention
from .mok import DeviceStatus
from .pipec2.launcher import Session

OUT_DIR = Path(__file__).resolve().parent / "stages" / "attention" / "out"
COMPOSITIONS = ("prefill", "prefill_softcap", "prefill_cp")
PARAMS = "<QiiiiQQfffiI4xQQQQQQQQiiiii4x"      # AttnParamsImage (stages/attention/attention.cuh), 152 bytes


def ensure_built() -> Path:
    if not all((OUT_DIR / c / f).exists() for c in COMPOSITIONS for f in ("pipeline.cubin", "one_tu.cubin", "link.json")):
        from .stages.attention import build
        build.build(OUT_DIR)
    return OUT_DIR


def _map(t: torch.Tensor) -> bytes:
    """[rows, heads, 128] bf16 as [rows, heads * 128]: box 128 rows x 64 columns, 128-byte swizzle."""
    buf = (ctypes.c_ubyte * 128)()
    _lib.call("plb_tensor_map_2d_bf16", buf, t.data_ptr(), t.shape[0], t.shape[1] * t.shape[2], 128, 64, 1)
    return bytes(buf)


class LinkedAttention:
    def __init__(self, out_dir=None, image: str = "pipeline.cubin"):
        """image: "pipeline.cubin" (linked) or "one_tu.cubin" (the single-unit build of the same sources)."""
        out = Path(out_dir or ensure_built())
        self.sessions = {c: Session(out / c, image) for c in COMPOSITIONS}

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, window: int = 0, softcap: float = 0.0,
                check: bool = True):
        """attention.attention_fwd for head pairs (an even number of query heads per KV head)."""
        B, S, Hq, d = q.shape
        Hkv = k.shape[2]
        if d != attention.D or S % attention.BLK or q.dtype != torch.bfloat16 or attention.heads_per_work(Hq, Hkv) != 2:
            raise ValueError("the linked images are the head-pair kernel: bf16, head_dim 128, S % 128 == 0, Hq / Hkv even")
        out = torch.empty_like(q)
        lse = torch.empty((B * Hq, S), dtype=torch.float32, device=q.device)
        work = attention._device_work(B, S, Hq, 2, window, q.device)
        status = DeviceStatus(q.device)
        # the scalars the library's launcher derives, in its single-precision arithmetic
        f32 = np.float32
        scale, log2e = f32(1.0 / math.sqrt(attention.D)), f32(1.4426950408889634)
        cap_in = float(scale / f32(softcap)) if softcap > 0 else 0.0
        s = self.sessions["prefill_softcap" if softcap > 0 else "prefill"]
        p = struct.pack(PARAMS, work.data_ptr(), work.shape[0], Hq, Hq // Hkv, S, out.data_ptr(), lse.data_ptr(),
                        float(scale * log2e), cap_in, float(f32(softcap) * log2e),
                        int(window), 0, 0, status.buf.data_ptr(), 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0)
        q2, k2, v2 = q.reshape(B * S, Hq, d), k.reshape(B * S, Hkv, d), v.reshape(B * S, Hkv, d)
        for stage_id in s.offsets:
            if stage_id.startswith("attn.load"):
                s.set_params(stage_id, _map(q2) + _map(k2) + _map(v2) + p)
            else:
                s.set_params(stage_id, p)
        sms = torch.cuda.get_device_properties(q.device).multi_processor_count
        s.launch((min(sms, work.shape[0]), 1, 1), torch.cuda.current_stream().cuda_stream)
        if check:
            status.check("linked attention")
        return out, lse

    def attend_and_push(self, rank, q_local: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor):
        """``CpRank.attend_and_push`` through the `prefill_cp` image: the gather owner's two warps push this
        rank's K/V blocks to the ranks that need them while the load owner acquires each key block's
        readiness counter. `rank` is an ``attention.CpRank`` (it owns the gathered buffers, counters,
        peers tables, ticket and work list); one launch, every CTA resident."""
        r = rank
        if r.step_heads != 2:
            raise ValueError("the linked images are the head-pair kernel")
        r.generation += r.PARTS
        r.ticket.zero_()
        f32 = np.float32
        block_bytes = attention.BLK * r.kv_heads * attention.D * 2
        s = self.sessions["prefill_cp"]
        p = struct.pack(PARAMS, r.work.data_ptr(), r.work.shape[0], r.q_heads, r.q_heads // r.kv_heads, 2 * r.C, r.out.data_ptr(),
                        r.lse.data_ptr(), float(f32(1.0 / math.sqrt(attention.D)) * f32(1.4426950408889634)), 0.0, 0.0, 0,
                        r.generation, r.ready.data_ptr(), r.status.buf.data_ptr(), k_local.data_ptr(), v_local.data_ptr(),
                        r.k_peers.data_ptr(), r.v_peers.data_ptr(), r.ready_peers.data_ptr(), r.ticket.data_ptr(),
                        r.C // attention.BLK, (block_bytes // r.PARTS) >> 4, r.PARTS, r.rank, r.world)
        for stage_id in s.offsets:
            if stage_id.startswith("attn.load"):
                s.set_params(stage_id, _map(q_local) + _map(r.k_gather) + _map(r.v_gather) + p)
            else:
                s.set_params(stage_id, p)
        sms = torch.cuda.get_device_properties(q_local.device).multi_processor_count
        s.launch((min(sms, r.work.shape[0]), 1, 1), torch.cuda.current_stream().cuda_stream)
        return r.out, r.lse

    def close(self):
        for s in self.sessions.values():
            s.close()
        self.sessions = {}
