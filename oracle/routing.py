"""CPU oracle for MoE routing and the padded expert schedule — TEST INFRASTRUCTURE.

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import this module.

Pinned by the reference tree: inputs are ``topk(randn logits)`` with router weights
``softmax(top-k values)`` and, every third generation, concentrated routing that leaves
experts empty (campaigns/mok/host/mok_port_host.py:273-282); every expert segment is padded
to EXPERT_PADDING rows (:93-96; campaigns/mok/port/framework/interp_fwd.cu:324); padding rows
carry ``peer_rank = -1``; the outputs compared bitwise are ``peer_rank``, ``peer_token_idx`` on
valid rows, ``num_tokens`` and ``tokens_per_expert`` (:356-363).

PARITY UNPINNED for the row order inside an expert segment: upstream
``functional.build_schedule`` / ``ops.schedule_out`` are in the absent submodule. This library
fixes it as ascending (source rank, token, slot).
"""
from __future__ import annotations

import numpy as np


def route_topk(logits: np.ndarray, topk: int):
    """top-k ids (ties: lower index first, descending value) and softmax over the selected logits."""
    logits = np.asarray(logits, dtype=np.float32)
    order = np.argsort(-logits, axis=1, kind="stable")[:, :topk]
    vals = np.take_along_axis(logits, order, axis=1)
    m = vals.max(axis=1, keepdims=True)
    ex = np.exp((vals - m).astype(np.float32)).astype(np.float32)
    w = (ex / ex.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)
    return order.astype(np.int32), w


def build_schedule(routes: np.ndarray, expert_base: int, num_local_experts: int, capacity: int,
                   padding: int = 128):
    """routes i32 [world, tokens, topk] -> dict of the arrays the device schedule writes."""
    routes = np.asarray(routes, dtype=np.int32)
    world, tokens, topk = routes.shape
    flat = routes.reshape(-1) - expert_base
    E = num_local_experts
    counts = np.array([(flat == e).sum() for e in range(E)], dtype=np.int32)
    padded = (counts + padding - 1) // padding * padding
    offsets = np.zeros(E + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(padded)
    total = int(offsets[E])
    if total > capacity:
        raise ValueError(f"{total} padded rows exceed capacity {capacity}")
    peer_rank = np.full(capacity, -1, dtype=np.int32)
    peer_token_idx = np.zeros(capacity, dtype=np.int32)
    dest_row = np.full(capacity, -1, dtype=np.int32)
    per_rank = tokens * topk
    for e in range(E):
        idx = np.nonzero(flat == e)[0]  # ascending = (rank, token, slot) order
        seg = slice(int(offsets[e]), int(offsets[e]) + len(idx))
        peer_rank[seg] = idx // per_rank
        rem = idx % per_rank
        peer_token_idx[seg] = rem // topk
        dest_row[seg] = rem
    block_expert = np.full(capacity // 128, -1, dtype=np.int32)
    for e in range(E):
        block_expert[offsets[e] // 128: offsets[e + 1] // 128] = e
    return dict(peer_rank=peer_rank, peer_token_idx=peer_token_idx, dest_row=dest_row,
                num_tokens=np.array([total], dtype=np.int32), tokens_per_expert=counts,
                expert_offsets=offsets, block_expert=block_expert)
