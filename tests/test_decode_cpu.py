"""Decode oracle and schedule builder, GPU-free."""
import math

import numpy as np
import pytest
import torch

from oracle import decode as od


def test_rope_tables_match_transformers_llama3():
    from transformers import LlamaConfig
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    rope = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
            "original_max_position_embeddings": 8192, "rope_theta": 500000.0}
    try:
        cfg = LlamaConfig(hidden_size=2048, num_attention_heads=32, head_dim=64, rope_theta=500000.0,
                          rope_scaling=dict(rope), max_position_embeddings=131072)
        inv, _ = ROPE_INIT_FUNCTIONS["llama3"](cfg, "cpu")
    except Exception as exc:  # signature drift between transformers versions
        pytest.skip(f"transformers rope helper unavailable: {exc}")
    cos, sin = od.rope_tables(64)
    ang = torch.arange(64, dtype=torch.float64)[:, None] * inv.double()[None, :]
    np.testing.assert_allclose(cos, torch.cos(ang).float().numpy(), rtol=0, atol=1e-5)
    np.testing.assert_allclose(sin, torch.sin(ang).float().numpy(), rtol=0, atol=1e-5)
    from pipelink_b200 import decode as hd
    c2, s2 = hd.rope_tables(64)
    assert np.array_equal(c2.numpy(), cos) and np.array_equal(s2.numpy(), sin)


def test_attention_oracle_partitions_merge_to_full():
    """LSE-weighted merge of the partial oracle equals unpartitioned attention."""
    rng = np.random.default_rng(0)
    q = rng.standard_normal((32, 64)) * 0.7
    k = rng.standard_normal((130, 8, 64)) * 0.7
    v = rng.standard_normal((130, 8, 64)) * 0.7
    full, full_lse = od.attention_partial_f64(q, k, v, 129, 1)
    for parts in (2, 3, 8, 24):
        out, lse = od.attention_partial_f64(q, k, v, 129, parts)
        out, lse = out.reshape(8, parts, 4, 64), lse.reshape(8, parts, 4)
        m = lse.max(axis=1, keepdims=True)
        w = np.where(np.isinf(lse), 0.0, np.exp2(lse - m))
        merged = (w[..., None] * out).sum(axis=1) / w.sum(axis=1)[..., None]
        np.testing.assert_allclose(merged.reshape(32, 64), full, rtol=1e-10, atol=1e-12)
        np.testing.assert_allclose((m[:, 0] + np.log2(w.sum(axis=1))).reshape(-1), full_lse, rtol=1e-12)
    # 24 partitions of 17 tokens: only the first two are non-empty
    out, lse = od.attention_partial_f64(q, k, v, 17, 24)
    assert np.isinf(lse.reshape(8, 24, 4)[:, 2:]).all() and (out.reshape(8, 24, 4, 64)[:, 2:] == 0).all()


@pytest.mark.parametrize("fuse", [True, False])
@pytest.mark.parametrize("num_sms,layers,vocab,parts", [(148, 16, 128256, 18), (148, 2, 1024, 3), (8, 1, 64, 1)])
def test_schedule_covers_every_row_once_and_counts_match(num_sms, layers, vocab, parts, fuse):
    from pipelink_b200 import decode as hd
    inst, nbars = hd.build_schedule(num_sms, layers, vocab, parts, fuse_reduce=fuse)
    assert inst.shape[0] == num_sms and inst.shape[2] == 32 and nbars == (layers + 1) * 8 + layers * 8
    rows = inst.reshape(-1, 32).numpy()
    rows = rows[rows[:, 0] != 0]
    signals = {}
    arrivals = {}
    for r in rows:
        if r[0] == 2 and r[5] > 0:
            # partitions count themselves in; only the last one bumps the counter of word 8
            assert (layers + 1) * 8 <= r[5] - 1 < nbars
            if r[5] not in arrivals:
                signals[r[8]] = signals.get(r[8], 0) + 1
            arrivals[r[5]] = arrivals.get(r[5], 0) + 1
            assert r[3] == parts
        elif r[8] >= 0:
            signals[r[8]] = signals.get(r[8], 0) + 1
    assert all(n == parts for n in arrivals.values()) and len(arrivals) == (layers * 8 if fuse else 0)
    for r in rows:
        if r[6] >= 0:
            assert signals[r[6]] == r[7], "a wait target must equal the number of producers"
    for l in range(layers):
        for op, total, unit in ((1, od.QKV_ROWS, 1), (4, od.HIDDEN, 1), (5, od.FFN, 1), (6, od.HIDDEN, 1)):
            sel = rows[(rows[:, 0] == op) & (rows[:, 1] == l)]
            cover = np.zeros(total, int)
            for r in sel:
                assert r[3] > 0 and (op == 5 or (r[2] % 2 == 0 and r[3] % 2 == 0))
                cover[r[2]: r[2] + r[3]] += 1
            assert (cover == 1).all()
        att = rows[(rows[:, 0] == 2) & (rows[:, 1] == l)]
        assert sorted((r[2], r[4]) for r in att) == [(h, p) for h in range(8) for p in range(parts)]
        red = rows[(rows[:, 0] == 3) & (rows[:, 1] == l)]
        assert sorted(r[2] for r in red) == ([] if fuse else list(range(0, 32, 4)))
    lm = rows[rows[:, 0] == 7]
    cover = np.zeros(vocab, int)
    for r in lm:
        cover[r[2]: r[2] + r[3]] += 1
    assert (cover == 1).all() and len(lm) == num_sms
    # program order on every SM follows the global op order, so the counters cannot deadlock
    for sm in range(num_sms):
        seq = [(r[1] if r[0] < 7 else layers, r[0]) for r in inst[sm].numpy() if r[0] != 0]
        assert seq == sorted(seq)


def test_decode_step_oracle_self_consistency():
    model = od.init_model(1, 512, seed=1)
    cos, sin = od.rope_tables(8)
    kc = np.zeros((1, 8, 8, 64), np.float32)
    vc = np.zeros_like(kc)
    h = model["lm_head"][5]
    r0 = od.decode_step(model, kc, vc, h, 0, cos, sin)
    # with a single position the attention output is exactly V of that position
    np.testing.assert_allclose(r0["attn_out"].reshape(8, 4, 64), np.repeat(vc[0, 0][:, None], 4, axis=1), atol=1e-6)
    assert r0["logits"].shape == (512,) and 0 <= r0["token"] < 512
    bad, _ = od.gate(r0["logits"], r0["logits"])
    assert bad == 0
