"""Host side of causal prefill attention and its context-parallel composition.

Single GPU: ``attention_fwd(q, k, v)`` builds the work list (one record per 128-query tile and
head, heavy tiles first) and calls ``plb_attention_fwd``.

Context parallel (the reference's ``cp`` composition, campaigns/attention/README.md:216-262):
the sequence is cut into 2W chunks, rank r owns chunks r and 2W-1-r (zigzag); queries never
move; every rank pushes its K/V blocks into the gathered, global-order buffers of the ranks that
need them (``plb_cp_push_kv``) and bumps one readiness counter per 128-token block; the attention
kernel's load lane acquires a block's counter right before its first TMA of that block. A step is
[group barrier] -> push -> attention, all on one stream: the push never waits on peers, so no two
kernels on one GPU wait on each other.
"""
from __future__ import annotations

import ctypes
import functools
import math

import numpy as np
import torch

from . import _lib
from .mok import DeviceStatus, _stream

BLK, D = 128, 128


def heads_per_work(q_heads: int, kv_heads: int) -> int:
    """2 when consecutive query heads pair up inside one KV group (one record, one K/V fetch for
    both), else 1."""
    return 2 if (q_heads // kv_heads) % 2 == 0 else 1


@functools.lru_cache(maxsize=64)
def _device_work(batch, seq, q_heads, step, window, device):
    return torch.from_numpy(causal_work(batch, seq, q_heads, step, window)).to(device)


def causal_work(batch: int, seq: int, q_heads: int, step: int = 1, window: int = 0) -> np.ndarray:
    """i32 [n, 8]: (q_row0, q_pos0, kv_row0, kv_pos0, kv_blocks, head, batch, 0), longest tiles first;
    one record per `step` consecutive heads. With a sliding window a tile starts at the block that
    holds the oldest key its first query still sees."""
    rows = []
    for qb in range(seq // BLK - 1, -1, -1):
        first = max(0, (qb * BLK - window + 1) // BLK) if window > 0 else 0
        for b in range(batch):
            for h in range(0, q_heads, step):
                rows.append((b * seq + qb * BLK, qb * BLK, b * seq + first * BLK, first * BLK, qb + 1 - first, h, b, 0))
    rows.sort(key=lambda r: -r[4])
    return np.asarray(rows, dtype=np.int32).reshape(-1, 8)


def zigzag_work(seq: int, world: int, rank: int, q_heads: int, step: int = 1) -> np.ndarray:
    """Work list of one rank (batch 1): local tile t covers global positions s*C + (128 t mod C),
    s = rank for the early chunk and 2W-1-rank for the late one (src/sm90/README.md:202-209)."""
    C = seq // (2 * world)
    items = []
    for t in range(2 * C // BLK):
        s = rank if t * BLK < C else 2 * world - 1 - rank
        pos = s * C + (t * BLK) % C
        items.append((pos, t))
    rows = []
    for pos, t in sorted(items, reverse=True):
        for h in range(0, q_heads, step):
            rows.append((t * BLK, pos, 0, 0, pos // BLK + 1, h, 0, 0))
    return np.asarray(rows, dtype=np.int32).reshape(-1, 8)


def _launch(q, k, v, out, lse, work, step, seq_q, ready, ready_target, status, window=0, softcap=0.0):
    q_rows, q_heads = q.shape[0], q.shape[1]
    kv_rows, kv_heads = k.shape[0], k.shape[1]
    _lib.call("plb_attention_fwd", q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
              work.data_ptr(), work.shape[0], step, q_heads, kv_heads, seq_q, q_rows, kv_rows, 1.0 / math.sqrt(D),
              int(window), float(softcap), 0 if ready is None else ready.data_ptr(), ready_target, status.buf.data_ptr(),
              _stream())


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, check: bool = True, pair_heads: bool | None = None,
                  window: int = 0, softcap: float = 0.0):
    """q [B, S, Hq, 128], k / v [B, S, Hkv, 128] bf16 CUDA. Returns (O like q, LSE f32 [B*Hq, S]).
    `pair_heads` None picks the two-heads-per-CTA kernel whenever Hq / Hkv is even. `window` > 0 adds
    the sliding-window mask (a query sees its last `window` keys), `softcap` > 0 the tanh soft cap
    on the scaled scores; both are the reference's mask / score stage variants."""
    B, S, Hq, d = q.shape
    if d != D or S % BLK or q.dtype != torch.bfloat16:
        raise ValueError("attention_fwd wants bf16, head_dim 128 and a sequence that is a multiple of 128")
    Hkv = k.shape[2]
    out = torch.empty_like(q)
    lse = torch.empty((B * Hq, S), dtype=torch.float32, device=q.device)
    step = heads_per_work(Hq, Hkv) if pair_heads is None else (2 if pair_heads else 1)
    work = _device_work(B, S, Hq, step, window, q.device)   # built once per shape and device
    status = DeviceStatus(q.device)
    _launch(q.reshape(B * S, Hq, D), k.reshape(B * S, Hkv, D), v.reshape(B * S, Hkv, D), out.reshape(B * S, Hq, D),
            lse, work, step, S, None, 0, status, window, softcap)
    if check:
        status.check("attention_fwd")
    return out, lse


class CpRank:
    """One rank of a context-parallel group (batch 1). Buffers peers write into (`k_gather`,
    `v_gather`, `ready`, barrier `flags`) live in a slab that is shared through CUDA IPC
    (``ep.IpcGroup``-style) or, for single-GPU tests, allocated side by side in one process."""

    PARTS = 8        # pieces a K/V block is pushed in by the gather warps of the attention launch

    def __init__(self, seq: int, q_heads: int, kv_heads: int, rank: int, world: int, slab_ptrs, layout, device,
                 fused_push: bool = False):
        """fused_push: the K/V exchange runs inside the attention launch (two gather warps per CTA)
        instead of as a launch in front of it. It needs head pairs, and ranks that are real GPUs:
        ranks emulated one after another on one GPU would wait for blocks that only a later launch
        pushes."""
        from .ep import barrier_state_for, tensor_from_ptr
        self.seq, self.rank, self.world, self.device = seq, rank, world, torch.device(device)
        self.C = seq // (2 * world)
        if self.C % BLK:
            raise ValueError("sequence / (2 * world) must be a multiple of 128")
        self.q_heads, self.kv_heads = q_heads, kv_heads
        dev = self.device
        me = slab_ptrs[rank]
        self.k_gather = tensor_from_ptr(me + layout["k"], (seq, kv_heads, D), torch.bfloat16, dev)
        self.v_gather = tensor_from_ptr(me + layout["v"], (seq, kv_heads, D), torch.bfloat16, dev)
        self.ready = tensor_from_ptr(me + layout["ready"], (seq // BLK,), torch.int32, dev)
        table = lambda off: torch.tensor([p + off for p in slab_ptrs], dtype=torch.int64, device=dev)
        self.k_peers, self.v_peers = table(layout["k"]), table(layout["v"])
        self.ready_peers, self.flags_peers = table(layout["ready"]), table(layout["flags"])
        self.step_heads = heads_per_work(q_heads, kv_heads)
        self.work = torch.from_numpy(zigzag_work(seq, world, rank, q_heads, self.step_heads)).to(dev)
        # a session opened on a slab that has been used before continues from the generation its
        # flags and readiness counters already hold (one session at a time per slab and rank)
        self.barrier_state = barrier_state_for(me + layout["flags"], rank, dev)
        self.status = DeviceStatus(dev)
        self.generation = int(self.ready.max().item())      # the value every needed counter holds after the last step
        self.fused_push = bool(fused_push)
        if self.fused_push and self.step_heads != 2:
            raise ValueError("the gather warps live in the two-heads-per-CTA kernel: q_heads / kv_heads must be even")
        self.ticket = torch.zeros(1, dtype=torch.int32, device=dev)
        self.out = torch.empty((2 * self.C, q_heads, D), dtype=torch.bfloat16, device=dev)
        self.lse = torch.empty((q_heads, 2 * self.C), dtype=torch.float32, device=dev)

    @staticmethod
    def slab_layout(seq: int, kv_heads: int):
        kv = seq * kv_heads * D * 2
        lay = {"flags": 0, "ready": 256, "k": 256 + (seq // BLK * 4 + 255) // 256 * 256}
        lay["v"] = lay["k"] + kv
        lay["nbytes"] = lay["v"] + kv
        return lay

    def barrier(self):
        _lib.call("plb_ep_barrier", self.flags_peers.data_ptr(), self.barrier_state.data_ptr(), self.rank, self.world,
                  self.status.buf.data_ptr(), _stream())

    def push(self, k_local: torch.Tensor, v_local: torch.Tensor, ctas: int = 32):
        """k_local / v_local bf16 [2C, kv_heads, 128]: this rank's early chunk then its late chunk."""
        self.generation += 1        # a separate push adds one per block
        _lib.call("plb_cp_push_kv", k_local.data_ptr(), v_local.data_ptr(), self.C // BLK, BLK * self.kv_heads * D * 2,
                  self.rank, self.world, self.k_peers.data_ptr(), self.v_peers.data_ptr(), self.ready_peers.data_ptr(),
                  ctas, _stream())

    def attend(self, q_local: torch.Tensor):
        _launch(q_local, self.k_gather, self.v_gather, self.out, self.lse, self.work, self.step_heads, 2 * self.C, self.ready,
                self.generation, self.status)
        return self.out, self.lse

    def attend_and_push(self, q_local, k_local, v_local):
        """One launch: the gather warps push this rank's K/V while the other warps attend."""
        self.generation += self.PARTS   # PARTS pieces per block
        _lib.call("plb_attention_fwd_cp", q_local.data_ptr(), self.k_gather.data_ptr(), self.v_gather.data_ptr(),
                  self.out.data_ptr(), self.lse.data_ptr(), self.work.data_ptr(), self.work.shape[0], self.q_heads,
                  self.kv_heads, 2 * self.C, q_local.shape[0], self.seq, 1.0 / math.sqrt(D), self.ready.data_ptr(),
                  self.generation, k_local.data_ptr(), v_local.data_ptr(), self.C // BLK, BLK * self.kv_heads * D * 2,
                  self.PARTS, self.rank, self.world, self.k_peers.data_ptr(), self.v_peers.data_ptr(),
                  self.ready_peers.data_ptr(), self.ticket.data_ptr(), self.status.buf.data_ptr(), _stream())
        return self.out, self.lse

    def step(self, q_local, k_local, v_local, distributed: bool = True):
        if distributed:
            self.barrier()       # every rank has finished reading the previous step's gathered K/V
        if self.fused_push:
            return self.attend_and_push(q_local, k_local, v_local)
        self.push(k_local, v_local)
        return self.attend(q_local)


def shard_zigzag(t: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """[S, ...] -> this rank's [2C, ...] (early chunk then late chunk)."""
    C = t.shape[0] // (2 * world)
    return torch.cat([t[rank * C:(rank + 1) * C], t[(2 * world - 1 - rank) * C:(2 * world - rank) * C]]).contiguous()
