"""CPU oracle for batch-1 Llama-shaped decode — TEST INFRASTRUCTURE, never on the product path.

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import
this module.

Pinned by the reference tree:
  * the partial-attention oracle: float64 restatement of
    campaigns/megakernel/host/check_cute_attention.cu:71-135 (16-token KV blocks, partition
    width ``ceil(ceil(len/16)/parts)*16``, scale 0.125, LSE in base 2, empty partition ->
    zeros / -inf, pass when ``|err| <= 0.02 (rms + |ref|)`` and ``|lse err| <= 2e-4``), on the
    same lengths x partitions grid and the same N(0, 0.7) bf16 inputs (its generator is
    ``std::mt19937`` + ``normal_distribution``, which is library-specific, so the seeded values
    here differ; the distribution and the predicate do not);
  * model shape, init and gates: campaigns/megakernel/host/export_inputs.py:96-119,146-157
    (N(0, 0.02) weights, norm weights 1, tied LM head, RoPE theta 5e5 with llama3 scaling,
    interleaved pairs), campaigns/megakernel/host/compare.py:30-31 (rtol 2e-2, atol 2e-2 * RMS).
PARITY UNPINNED for the op arithmetic other than attention: the reference's PyVM and op bodies
are in the absent ``HazyResearch/Megakernels`` submodule; this restates the published Llama
forward with bf16 rounding wherever the reference stores bf16 (hidden, q, k, v, attn_out,
silu_out, logits).
"""
from __future__ import annotations

import math

import numpy as np

from .mxfp8 import bf16_round

HIDDEN, Q_HEADS, KV_HEADS, HEAD_DIM, FFN = 2048, 32, 8, 64, 8192
QKV_ROWS = (Q_HEADS + 2 * KV_HEADS) * HEAD_DIM
EPS = 1e-5
ATTN_SCALE = 1.0 / math.sqrt(HEAD_DIM)


def rope_tables(rows: int, theta: float = 500000.0, factor: float = 32.0, low: float = 1.0,
                high: float = 4.0, original: int = 8192):
    """cos/sin f32 [rows, 32]: one angle per rotated pair, llama3 frequency scaling."""
    i = np.arange(HEAD_DIM // 2, dtype=np.float64)
    inv = 1.0 / theta ** (2.0 * i / HEAD_DIM)
    wavelen = 2.0 * math.pi / inv
    low_wl, high_wl = original / low, original / high
    smooth = (original / wavelen - low) / (high - low)
    scaled = np.where(wavelen > low_wl, inv / factor,
                      np.where(wavelen < high_wl, inv, (1 - smooth) * inv / factor + smooth * inv))
    ang = np.arange(rows, dtype=np.float64)[:, None] * scaled[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def init_model(layers: int, vocab: int, seed: int = 0):
    rng = np.random.default_rng(seed)
    w = lambda *shape: bf16_round(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))
    return dict(qkv_w=w(layers, QKV_ROWS, HIDDEN), o_w=w(layers, HIDDEN, HIDDEN), up_w=w(layers, FFN, HIDDEN),
                gate_w=w(layers, FFN, HIDDEN), down_w=w(layers, HIDDEN, FFN),
                attn_norm=np.ones((layers, HIDDEN), np.float32), mlp_norm=np.ones((layers, HIDDEN), np.float32),
                lm_norm=np.ones(HIDDEN, np.float32), lm_head=w(vocab, HIDDEN))


def rms_norm(x, w):
    x = x.astype(np.float32)
    inv = np.float32(1.0) / np.sqrt(np.mean(x * x, dtype=np.float32) + np.float32(EPS))
    return (x * inv * w).astype(np.float32)


def partition_range(length, partitions, part):
    blocks = (length + 15) // 16
    per = (blocks + partitions - 1) // partitions
    begin = part * per * 16
    end = min(length, begin + per * 16)
    return min(begin, end), end


def attention_partial_f64(q, k, v, length, partitions, scale=0.125):
    """q [32,64], k/v [>=length, 8, 64] -> out f64 [(head*parts+part)*4+h, 64], lse2 f64."""
    out = np.zeros((KV_HEADS * partitions * 4, HEAD_DIM))
    lse = np.full(KV_HEADS * partitions * 4, -np.inf)
    q, k, v = q.astype(np.float64), k.astype(np.float64), v.astype(np.float64)
    for head in range(KV_HEADS):
        for part in range(partitions):
            b, e = partition_range(length, partitions, part)
            if b >= e:
                continue
            for h in range(4):
                idx = (head * partitions + part) * 4 + h
                s = (k[b:e, head] @ q[head * 4 + h]) * scale
                m = s.max()
                p = np.exp(s - m)
                out[idx] = (p @ v[b:e, head]) / p.sum()
                lse[idx] = (m + math.log(p.sum())) / math.log(2.0)
    return out, lse


def attention_gate(expected, expected_lse, got, got_lse):
    """The reference checker's predicate; returns the number of failing values."""
    fails = 0
    for idx in range(expected.shape[0]):
        if expected_lse[idx] == -np.inf:
            fails += int(got_lse[idx] != -np.inf) + int((got[idx] != 0).sum())
            continue
        rms = math.sqrt((expected[idx] ** 2).mean())
        err = np.abs(got[idx] - expected[idx])
        fails += int((~np.isfinite(got[idx]) | (err > 0.02 * (rms + np.abs(expected[idx])))).sum())
        fails += int(not np.isfinite(got_lse[idx]) or abs(got_lse[idx] - expected_lse[idx]) > 2e-4)
    return fails


def decode_step(model, k_cache, v_cache, hidden, pos, cos, sin, layers=None):
    """One token. hidden fp32 [2048] (bf16 values); caches fp32 [layers, max_seq, 8, 64] are
    updated in place at row ``pos``. Returns dict of the tensors the reference compares."""
    L = layers or model["qkv_w"].shape[0]
    hidden = hidden.astype(np.float32).copy()
    rec = {}
    for l in range(L):
        x = rms_norm(hidden, model["attn_norm"][l])
        qkv = model["qkv_w"][l] @ x
        c, s = cos[pos], sin[pos]
        rot = qkv[: (Q_HEADS + KV_HEADS) * HEAD_DIM].reshape(-1, HEAD_DIM // 2, 2)
        r0 = rot[:, :, 0] * c - rot[:, :, 1] * s
        r1 = rot[:, :, 1] * c + rot[:, :, 0] * s
        roped = bf16_round(np.stack([r0, r1], axis=-1).reshape(-1))
        q = roped[: Q_HEADS * HEAD_DIM].reshape(Q_HEADS, HEAD_DIM)
        k_cache[l, pos] = roped[Q_HEADS * HEAD_DIM:].reshape(KV_HEADS, HEAD_DIM)
        v_cache[l, pos] = bf16_round(qkv[(Q_HEADS + KV_HEADS) * HEAD_DIM:]).reshape(KV_HEADS, HEAD_DIM)
        attn = np.zeros((Q_HEADS, HEAD_DIM), np.float32)
        for kvh in range(KV_HEADS):
            K = k_cache[l, : pos + 1, kvh].astype(np.float64)
            V = v_cache[l, : pos + 1, kvh].astype(np.float64)
            for h in range(4):
                sc = (K @ q[kvh * 4 + h].astype(np.float64)) * ATTN_SCALE
                p = np.exp(sc - sc.max())
                attn[kvh * 4 + h] = (p @ V) / p.sum()
        attn_out = bf16_round(attn.reshape(-1))
        hidden = bf16_round(hidden + model["o_w"][l] @ attn_out)
        x = rms_norm(hidden, model["mlp_norm"][l])
        g = model["gate_w"][l] @ x
        u = model["up_w"][l] @ x
        silu = bf16_round((g / (np.float32(1.0) + np.exp(-g))) * u)
        hidden = bf16_round(hidden + model["down_w"][l] @ silu)
        if l == 0:
            rec.update(q_post_rope=q.reshape(-1).copy(), attn_out_l0=attn_out.copy(), silu_out_l0=silu.copy())
    x = rms_norm(hidden, model["lm_norm"])
    logits = bf16_round(model["lm_head"] @ x)
    token = int(np.argmax(logits))  # first maximum = lowest id on ties
    rec.update(hidden_states=hidden, logits=logits, token=token, q_last=q.reshape(-1), attn_out=attn_out,
               silu_out=silu, k_row=k_cache[L - 1, pos].reshape(-1).copy(), v_row=v_cache[L - 1, pos].reshape(-1).copy())
    return rec


def gate(reference, actual, rtol=2e-2, atol_rms=2e-2):
    """compare.py's allclose gate: |a - r| <= atol + rtol |r| with atol = atol_rms * RMS(ref)."""
    r = np.asarray(reference, np.float64).reshape(-1)
    a = np.asarray(actual, np.float64).reshape(-1)
    atol = atol_rms * math.sqrt((r * r).mean())
    bad = np.abs(a - r) > atol + rtol * np.abs(r)
    return int(bad.sum()), float(np.abs(a - r).max())
