"""CPU oracle for causal prefill attention — TEST INFRASTRUCTURE, never on the product path.

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import
this module.

Pinned by the reference tree:
  * inputs: Philox4x32-10 words (evaluator/harness/parity/streams.py:127-215; known answer
    ``philox4x32_10((0,0,0,0),(0,0)) = (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)``,
    evaluator/harness/parity/tests/test_parity.py:97-101), addressed as in
    campaigns/attention/src/slot/fixtures.cuh:52-102: key (0x50495045, 2), counter
    (block lo, block hi, numeric_case, role), value = bf16(-2 + 4 (word + 0.5) 2^-32);
  * the spot oracle: campaigns/attention/src/slot/family.cuh:156-229 - full visible keys for the
    sampled rows, LSE = max + log(sum) in natural log of the scaled scores;
  * the predicate: ``|a - r| <= 0.02 + 0.02 |r|``, ``-inf`` exact (fixtures.cuh:106-110).
"""
from __future__ import annotations

import math

import numpy as np

from .mxfp8 import bf16_round

M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
SEED, NAMESPACE_ATTENTION = 0x50495045, 2


def philox4x32_10(counter, key):
    """counter: 4 uint32 arrays (or ints), key: 2 ints -> 4 uint32 arrays."""
    v = [np.asarray(c, dtype=np.uint64) & 0xFFFFFFFF for c in counter]
    k0, k1 = key[0] & 0xFFFFFFFF, key[1] & 0xFFFFFFFF
    for _ in range(10):
        p0 = np.uint64(M0) * v[0]
        p1 = np.uint64(M1) * v[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & np.uint64(0xFFFFFFFF)
        hi1, lo1 = p1 >> np.uint64(32), p1 & np.uint64(0xFFFFFFFF)
        v = [(hi1 ^ v[1] ^ np.uint64(k0)) & np.uint64(0xFFFFFFFF), lo1,
             (hi0 ^ v[3] ^ np.uint64(k1)) & np.uint64(0xFFFFFFFF), lo0]
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return tuple(x.astype(np.uint32) for x in v)


def philox_bf16(count: int, numeric_case: int, role: int) -> np.ndarray:
    """fill_philox_bf16: element j uses word (j & 3) of block j >> 2. Returns fp32 (bf16 values)."""
    blocks = np.arange((count + 3) // 4, dtype=np.uint64)
    zeros = np.zeros_like(blocks)
    w = philox4x32_10((blocks & np.uint64(0xFFFFFFFF), blocks >> np.uint64(32), zeros + np.uint64(numeric_case),
                       zeros + np.uint64(role)), (SEED, NAMESPACE_ATTENTION))
    words = np.stack(w, axis=1).reshape(-1)[:count].astype(np.float64)
    u = (words + 0.5) * 2.0 ** -32
    return bf16_round((-2.0 + 4.0 * u).astype(np.float32))


def reference_rows(q, k, v, rows, scale, q_pos=None, window=0, softcap=0.0):
    """q [Sq, Hq, D], k/v [Sk, Hkv, D] fp32; rows = query rows to evaluate; q_pos[r] = global
    position of query r (defaults to r). Returns (out [len(rows), Hq, D], lse [Hq, len(rows)]).
    window > 0 keeps keys with kv_pos > q_pos - window (campaigns/attention/src/sm90/stage_mask_window.cu:8-11);
    softcap > 0 replaces the scaled score by softcap * tanh(score / softcap)
    (stage_score_softcap.cu:10-13 with family_params.cuh:112-113)."""
    Sq, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    out = np.zeros((len(rows), Hq, D), np.float64)
    lse = np.zeros((Hq, len(rows)), np.float64)
    for i, r in enumerate(rows):
        pos = r if q_pos is None else int(q_pos[r])
        for h in range(Hq):
            first = max(0, pos - window + 1) if window > 0 else 0
            s = (k[first: pos + 1, h // g].astype(np.float64) @ q[r, h].astype(np.float64)) * scale
            if softcap > 0:
                s = softcap * np.tanh(s / softcap)
            m = s.max()
            p = np.exp(s - m)
            out[i, h] = (p @ v[first: pos + 1, h // g].astype(np.float64)) / p.sum()
            lse[h, i] = m + math.log(p.sum())
    return out, lse


def matches(actual, reference):
    """The reference predicate; returns the number of violating values."""
    a, r = np.asarray(actual, np.float64), np.asarray(reference, np.float64)
    inf = np.isneginf(r)
    bad = np.where(inf, ~np.isneginf(a), ~(np.isfinite(a) & np.isfinite(r) & (np.abs(a - r) <= 0.02 + 0.02 * np.abs(r))))
    return int(bad.sum())


def boundary_rows(seq: int, extra=()):
    """Rows at tile boundaries plus a few interior ones (the reference samples boundary rows)."""
    rows = {0, 1, seq - 1}
    for b in range(128, seq, max(128, seq // 8 // 128 * 128)):
        rows.update((b - 1, b, b + 1))
    rows.update(extra)
    return sorted(r for r in rows if 0 <= r < seq)


def zigzag_rows(seq: int, world: int, rank: int):
    """Global positions owned by `rank`: chunks rank and 2W-1-rank of 2W equal chunks
    (campaigns/attention/README.md:222-228)."""
    c = seq // (2 * world)
    return np.concatenate([np.arange(rank * c, (rank + 1) * c), np.arange((2 * world - 1 - rank) * c, (2 * world - rank) * c)])
