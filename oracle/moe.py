"""CPU oracle for the MXFP8 MoE FFN forward — TEST INFRASTRUCTURE, never on the product path.

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import this module.

Follows the data flow of the reference's forward pass: dispatch quantises each scheduled
token row (campaigns/mok/port/comm/comm.cu:105-123); gate and up projections produce bf16
(campaigns/mok/port/gemm/gemm.cu:150-157); ``hidden = silu(gate) * up`` rounded to bf16 and
requantised along the intermediate dimension (campaigns/mok/port/act/act.cu:100-178); the down
projection writes bf16 rows that the combine stage places at ``token * k + slot``
(gemm.cu:158-162, comm.cu:124-129); the epilogue forms
``out = y_shared + sum_j w[t, j] * combine[t * k + j]`` (campaigns/mok/host/mok_port_host.py:204).

PARITY UNPINNED for tolerances and quantisation arithmetic (``tests.utils.MXFP8_TOLERANCE``,
``run_forward_reference_bf16`` and ``mxfp8.cuh`` are in absent submodules). Metrics follow
``error_stats`` (mok_port_host.py:292-306): abs-mean, abs-max, relative = sum|err| / sum|ref|.
"""
from __future__ import annotations

import numpy as np
import torch

from . import mxfp8


def _mm(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """fp32 a @ b.T on the host cores."""
    return torch.matmul(torch.from_numpy(np.ascontiguousarray(a)),
                        torch.from_numpy(np.ascontiguousarray(b)).T).numpy()


def silu_mul(gate: np.ndarray, up: np.ndarray, limit: float = 0.0) -> np.ndarray:
    """silu(gate) * up; with limit > 0 the clamped variant: gate bounded from above, up from both
    sides (campaigns/mok/port/act_gptoss/swiglu.cuh:143-147 applies the same bounds)."""
    g = gate.astype(np.float32)
    if limit > 0:
        g = np.minimum(g, np.float32(limit))
        up = np.clip(up.astype(np.float32), np.float32(-limit), np.float32(limit))
    s = (g / (np.float32(1.0) + np.exp(-g, dtype=np.float32))).astype(np.float32)
    return (s * up.astype(np.float32)).astype(np.float32)


def quantize_weights(w_gate, w_up, w_down):
    """bf16-representable fp32 [E, I, H] / [E, I, H] / [E, H, I] -> per-expert (fp8, sc) lists."""
    out = {}
    for name, w in (("gate", w_gate), ("up", w_up), ("down", w_down)):
        E, R, C = w.shape
        q, sc = mxfp8.quantize(w.reshape(E * R, C))
        out[name] = (q.reshape(E, R, C), sc)
    return out


def pack_gate_up(gate_q, gate_sc, up_q, up_sc, block=128):
    """Row interleave used by the fused gate/up GEMM: per expert `block` gate rows, `block` up rows, ..."""
    E, I, H = gate_q.shape
    B = block
    g_s = mxfp8.unpack_scales(gate_sc, E * I, H).reshape(E, I // B, B, H // 32)
    u_s = mxfp8.unpack_scales(up_sc, E * I, H).reshape(E, I // B, B, H // 32)
    q = np.stack([gate_q.reshape(E, I // B, B, H), up_q.reshape(E, I // B, B, H)], axis=2)
    s = np.stack([g_s, u_s], axis=2)
    return q.reshape(E, 2 * I, H), mxfp8.pack_scales(s.reshape(E * 2 * I, H // 32))


def dispatch(x_by_rank, sched):
    """Gather + quantise the scheduled rows. x_by_rank: list of fp32 [tokens, H] (bf16 values)."""
    total = int(sched["num_tokens"][0])
    H = x_by_rank[0].shape[1]
    rows = np.zeros((total, H), dtype=np.float32)
    pr, pt = sched["peer_rank"][:total], sched["peer_token_idx"][:total]
    for r, x in enumerate(x_by_rank):
        sel = pr == r
        rows[sel] = x[pt[sel]]
    q, sc = mxfp8.quantize(rows)
    return q, sc


def expert_ffn(xq, xsc, weights, sched, round_gate_up=True, context=None, limit=0.0):
    """Rows [total, H] quantised -> (hidden_q, hidden_sc, y bf16-valued fp32 [total, H]).
    `context` (a dict) receives the bf16 gate / up / hidden the backward pass differentiates through."""
    total, H = xq.shape
    gate_q, gate_sc = weights["gate"]
    up_q, up_sc = weights["up"]
    down_q, down_sc = weights["down"]
    E, I, _ = gate_q.shape
    x = mxfp8.dequantize(xq, xsc)
    wg = mxfp8.dequantize(gate_q.reshape(E * I, H), gate_sc).reshape(E, I, H)
    wu = mxfp8.dequantize(up_q.reshape(E * I, H), up_sc).reshape(E, I, H)
    wd = mxfp8.dequantize(down_q.reshape(E * H, I), down_sc).reshape(E, H, I)
    off = sched["expert_offsets"]
    hidden = np.zeros((total, I), dtype=np.float32)
    gate_all, up_all = np.zeros((total, I), dtype=np.float32), np.zeros((total, I), dtype=np.float32)
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi == lo:
            continue
        g = _mm(x[lo:hi], wg[e])
        u = _mm(x[lo:hi], wu[e])
        if round_gate_up:
            g, u = mxfp8.bf16_round(g), mxfp8.bf16_round(u)
        gate_all[lo:hi], up_all[lo:hi] = g, u
        hidden[lo:hi] = mxfp8.bf16_round(silu_mul(g, u, limit))
    if context is not None:
        context.update(gate=gate_all, up=up_all, hidden=hidden.copy())
    hq, hsc = mxfp8.quantize(hidden)
    hd = mxfp8.dequantize(hq, hsc)
    y = np.zeros((total, H), dtype=np.float32)
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi > lo:
            y[lo:hi] = mxfp8.bf16_round(_mm(hd[lo:hi], wd[e]))
    return hq, hsc, y


def combine(y, sched, rank, tokens, topk):
    """Place rows owned by `rank` at token * k + slot (rows from other ranks are ignored)."""
    total = int(sched["num_tokens"][0])
    H = y.shape[1]
    buf = np.zeros((tokens * topk, H), dtype=np.float32)
    pr, dr = sched["peer_rank"][:total], sched["dest_row"][:total]
    sel = pr == rank
    buf[dr[sel]] = y[:total][sel]
    return buf


def fwd_epilogue(combine_buf, router_w, y_shared=None):
    """out[t] = y_shared[t] + sum_j w[t, j] * combine[t*k + j]; separate fp32 roundings, j ascending."""
    tokens, topk = router_w.shape
    H = combine_buf.shape[1]
    c = combine_buf.reshape(tokens, topk, H).astype(np.float32)
    acc = np.zeros((tokens, H), dtype=np.float32) if y_shared is None else y_shared.astype(np.float32).copy()
    for j in range(topk):
        prod = (router_w[:, j:j + 1].astype(np.float32) * c[:, j]).astype(np.float32)
        acc = (acc + prod).astype(np.float32)
    return mxfp8.bf16_round(acc)


def forward_single_rank(x, routes, router_w, weights, padding=128, capacity=None, context=None, limit=0.0):
    """Whole forward on one rank. x fp32 (bf16 values) [T, H]; routes i32 [T, k]."""
    from . import routing
    T, k = routes.shape
    E = weights["gate"][0].shape[0]
    if capacity is None:
        capacity = ((T * k + E * (padding - 1)) + 127) // 128 * 128
    sched = routing.build_schedule(routes[None], 0, E, capacity, padding)
    xq, xsc = dispatch([x], sched)
    hq, hsc, y = expert_ffn(xq, xsc, weights, sched, context=context, limit=limit)
    buf = combine(y, sched, 0, T, k)
    out = fwd_epilogue(buf, router_w)
    return dict(schedule=sched, x_routed=(xq, xsc), hidden=(hq, hsc), y=y, combine=buf, output=out)


def forward_single_rank_bf16(x, routes, router_w, w_gate, w_up, w_down, padding=128, capacity=None, limit=0.0,
                             context=None):
    """Forward with the bf16 routed precision (the reference's second precision value,
    campaigns/mok/port/act/act.cu:246-249): no quantisation on the routed path; gate / up and the
    hidden rows are rounded to bf16 where the reference's bf16 tensors hold them
    (campaigns/mok/port/act_gptoss/swiglu.cuh:138-156), GEMMs accumulate in fp32.
    x fp32 (bf16 values) [T, H]; weights bf16-valued fp32 [E, I, H], [E, I, H], [E, H, I]."""
    from . import routing
    T, k = routes.shape
    E, I, H = w_gate.shape
    if capacity is None:
        capacity = ((T * k + E * (padding - 1)) + 127) // 128 * 128
    sched = routing.build_schedule(routes[None], 0, E, capacity, padding)
    total = int(sched["num_tokens"][0])
    pr, pt, off = sched["peer_rank"][:total], sched["peer_token_idx"][:total], sched["expert_offsets"]
    rows = np.zeros((total, H), np.float32)
    rows[pr >= 0] = x[pt[pr >= 0]]
    hidden = np.zeros((total, I), np.float32)
    gate_all, up_all = np.zeros((total, I), np.float32), np.zeros((total, I), np.float32)
    y = np.zeros((total, H), np.float32)
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi > lo:
            g, u = mxfp8.bf16_round(_mm(rows[lo:hi], w_gate[e])), mxfp8.bf16_round(_mm(rows[lo:hi], w_up[e]))
            gate_all[lo:hi], up_all[lo:hi] = g, u
            hidden[lo:hi] = mxfp8.bf16_round(silu_mul(g, u, limit))
            y[lo:hi] = mxfp8.bf16_round(_mm(hidden[lo:hi], w_down[e]))
    if context is not None:
        context.update(gate=gate_all, up=up_all, hidden=hidden.copy())
    buf = combine(y, sched, 0, T, k)
    return dict(schedule=sched, x_routed=rows, hidden=hidden, y=y, combine=buf, output=fwd_epilogue(buf, router_w))


def _pad_rows(a: np.ndarray, multiple: int = 128) -> np.ndarray:
    pad = (-a.shape[0]) % multiple
    return a if pad == 0 else np.concatenate([a, np.zeros((pad, a.shape[1]), dtype=a.dtype)])


def forward_token_rows(x_rows, routes, router_w, expert_weights, limit=0.0):
    """Spot rows of the forward pass: the outputs of a few tokens of a problem too large to run
    whole on the host (the method of the reference's own large cases, which check boundary rows
    only: campaigns/attention/src/slot/family.cuh:156-229). Every step of the path is local to a
    row (quantisation blocks run along a row, a GEMM row needs its own operand row and the
    expert's weights, the epilogue sums one token's slots), so the rows need no schedule.

    x_rows fp32 (bf16 values) [n, H]; routes i32 [n, k] global expert ids; router_w fp32 [n, k];
    expert_weights(e) -> ((gate_q, gate_sc), (up_q, up_sc), (down_q, down_sc)) of expert e, each
    quantised as quantize() writes a [rows, cols] matrix. Returns bf16-valued fp32 [n, H]."""
    n, H = x_rows.shape
    k = routes.shape[1]
    xq, xsc = mxfp8.quantize(_pad_rows(np.asarray(x_rows, dtype=np.float32)))
    xd = mxfp8.dequantize(xq, xsc)[:n]
    y = np.zeros((n * k, H), dtype=np.float32)
    for e in np.unique(routes):
        tok, slot = np.nonzero(routes == e)
        (gq, gsc), (uq, usc), (dq, dsc) = expert_weights(int(e))
        wg, wu, wd = mxfp8.dequantize(gq, gsc), mxfp8.dequantize(uq, usc), mxfp8.dequantize(dq, dsc)
        g = mxfp8.bf16_round(_mm(xd[tok], wg))
        u = mxfp8.bf16_round(_mm(xd[tok], wu))
        hidden = _pad_rows(mxfp8.bf16_round(silu_mul(g, u, limit)))
        hd = mxfp8.dequantize(*mxfp8.quantize(hidden))[:len(tok)]
        y[tok * k + slot] = mxfp8.bf16_round(_mm(hd, wd))
    return fwd_epilogue(y, np.asarray(router_w, dtype=np.float32))


def error_stats(expected, actual):
    """abs-mean, abs-max, relative (= sum|err| / sum|ref|), and relative L2."""
    e = np.asarray(expected, dtype=np.float64).reshape(-1)
    a = np.asarray(actual, dtype=np.float64).reshape(-1)
    d = np.abs(e - a)
    return dict(abs_mean=float(d.mean()), abs_max=float(d.max()),
                relative=float(d.sum() / max(np.abs(e).sum(), 1e-300)),
                rel_l2=float(np.sqrt((d * d).sum() / max((e * e).sum(), 1e-300))))


def forward_multi_rank(xs, routes, router_ws, weights, world, padding=128):
    """Expert-parallel forward: xs[r] fp32 [T, H], routes[r] i32 [T, k] (global expert ids),
    router_ws[r] fp32 [T, k]; `weights` holds all experts, rank r owns a contiguous slice.
    Returns per-rank outputs plus the per-rank schedules and combine buffers."""
    from . import routing
    T, k = routes[0].shape
    E = weights["gate"][0].shape[0]
    El = E // world
    gathered = np.stack(routes).astype(np.int32)
    combine_bufs = [np.zeros((T * k, xs[0].shape[1]), dtype=np.float32) for _ in range(world)]
    scheds, hiddens = [], []
    for r in range(world):
        cap = ((world * T * k + El * (padding - 1)) + 127) // 128 * 128
        sched = routing.build_schedule(gathered, r * El, El, cap, padding)
        local = {}
        for name in ("gate", "up", "down"):
            q, sc = weights[name]
            rows, cols = q.shape[1], q.shape[2]
            sc_rg = mxfp8.unpack_scales(sc, E * rows, cols).reshape(E, rows, cols // 32)
            local[name] = (q[r * El:(r + 1) * El],
                           mxfp8.pack_scales(sc_rg[r * El:(r + 1) * El].reshape(El * rows, cols // 32)))
        xq, xsc = dispatch(xs, sched)
        hq, hsc, y = expert_ffn(xq, xsc, local, sched)
        total = int(sched["num_tokens"][0])
        pr, dr = sched["peer_rank"][:total], sched["dest_row"][:total]
        for home in range(world):
            sel = pr == home
            combine_bufs[home][dr[sel]] = y[:total][sel]
        scheds.append(sched)
        hiddens.append((hq, hsc))
    outs = [fwd_epilogue(combine_bufs[r], router_ws[r]) for r in range(world)]
    return dict(outputs=outs, schedules=scheds, combine=combine_bufs, hidden=hiddens)


def _deq_t(a):
    """Transposed quantisation of a [R, C] -> dequantised [C, R]."""
    return mxfp8.dequantize(*mxfp8.quantize_transposed(a))


def backward_single_rank(x, router_w, w_gate, w_up, w_down, fwd, ctx, d_out, limit=0.0):
    """Backward of forward_single_rank with the same quantisation points as the device path:
    d_y, d_hidden and [d_gate | d_up] are bf16 tensors quantised along the contraction dimension of
    each GEMM that consumes them (normal orientation for data gradients, transposed for weight
    gradients); weights enter the data gradients transposed-quantised
    (campaigns/mok/port/gemm/gemm.cu:166-243, campaigns/mok/host/resources.py:62-77).
    x, d_out fp32 [T, H]; w_* bf16-valued fp32; fwd / ctx from forward_single_rank(context=ctx)."""
    sched = fwd["schedule"]
    total = int(sched["num_tokens"][0])
    off, pr, pt, dr = sched["expert_offsets"], sched["peer_rank"][:total], sched["peer_token_idx"][:total], sched["dest_row"][:total]
    T, k = router_w.shape
    E, I, H = w_gate.shape
    live = pr >= 0
    wflat = router_w.reshape(-1).astype(np.float32)
    dy = np.zeros((total, H), np.float32)
    dy[live] = mxfp8.bf16_round((wflat[dr[live]][:, None] * d_out[pt[live]]).astype(np.float32))
    d_router = np.zeros(T * k, np.float32)
    d_router[dr[live]] = (d_out[pt[live]].astype(np.float64) * fwd["combine"][dr[live]].astype(np.float64)).sum(axis=1)
    dyd = mxfp8.dequantize(*mxfp8.quantize(dy))
    dy_t, hid_t = _deq_t(dy), _deq_t(ctx["hidden"])
    d_hidden = np.zeros((total, I), np.float32)
    d_w_down = np.zeros((E, H, I), np.float32)
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi > lo:
            d_hidden[lo:hi] = mxfp8.bf16_round(_mm(dyd[lo:hi], _deq_t(w_down[e])))          # [rows, H] x [I, H]^T
            d_w_down[e] = mxfp8.bf16_round(_mm(dy_t[:, lo:hi], hid_t[:, lo:hi]))            # [H, rows] x [I, rows]^T
    g = mxfp8.dequantize(*mxfp8.quantize(ctx["gate"]))
    u = mxfp8.dequantize(*mxfp8.quantize(ctx["up"]))
    g_open, u_open = np.ones_like(g, dtype=bool), np.ones_like(u, dtype=bool)
    if limit > 0:
        # no gradient through a bound that is active or met with equality (swiglu.cuh:13-21,29-37)
        lim = np.float32(limit)
        g_open, u_open = g < lim, (u > -lim) & (u < lim)
        g, u = np.minimum(g, lim), np.clip(u, -lim, lim)
    sg = (np.float32(1.0) / (np.float32(1.0) + np.exp(-g))).astype(np.float32)
    d_up = np.where(u_open, d_hidden * (g * sg), np.float32(0.0))
    d_gate = np.where(g_open, d_hidden * u * sg * (np.float32(1.0) + g * (np.float32(1.0) - sg)), np.float32(0.0))
    dgu = mxfp8.bf16_round(np.concatenate([d_gate, d_up], axis=1).astype(np.float32))
    dgud = mxfp8.dequantize(*mxfp8.quantize(dgu))
    rows = np.zeros((total, H), np.float32)
    rows[live] = x[pt[live]]
    dgu_t, x_t = _deq_t(dgu), _deq_t(rows)
    d_x_buf = np.zeros((T * k, H), np.float32)
    d_w_cat = np.zeros((E, 2 * I, H), np.float32)
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi > lo:
            dxr = mxfp8.bf16_round(_mm(dgud[lo:hi], _deq_t(np.concatenate([w_gate[e], w_up[e]]))))   # [rows, 2I] x [H, 2I]^T
            sel = pr[lo:hi] >= 0
            d_x_buf[dr[lo:hi][sel]] = dxr[sel]
            d_w_cat[e] = mxfp8.bf16_round(_mm(dgu_t[:, lo:hi], x_t[:, lo:hi]))                       # [2I, rows] x [H, rows]^T
    d_x = fwd_epilogue(d_x_buf, np.ones((T, k), np.float32))
    return dict(d_x=d_x, d_router_weights=d_router.reshape(T, k), d_w_routed_gate=d_w_cat[:, :I], d_w_routed_up=d_w_cat[:, I:],
                d_w_routed_down=d_w_down, d_hidden=d_hidden, d_gate_up=dgu, d_y=dy)


def backward_single_rank_bf16(x, router_w, w_gate, w_up, w_down, fwd, ctx, d_out, limit=0.0):
    """Backward of forward_single_rank_bf16 (the bwd / rec cells of the bf16 routed precision,
    campaigns/mok/README.md:86-104): the pass structure of backward_single_rank
    (campaigns/mok/port/gemm/gemm.cu:166-243) with no quantisation: every GEMM takes the bf16 tensors
    themselves, accumulates in fp32 and its result is rounded to bf16 where a bf16 tensor holds it."""
    sched = fwd["schedule"]
    total = int(sched["num_tokens"][0])
    off, pr, pt, dr = sched["expert_offsets"], sched["peer_rank"][:total], sched["peer_token_idx"][:total], sched["dest_row"][:total]
    T, k = router_w.shape
    E, I, H = w_gate.shape
    live = pr >= 0
    wflat = router_w.reshape(-1).astype(np.float32)
    dy = np.zeros((total, H), np.float32)
    dy[live] = mxfp8.bf16_round((wflat[dr[live]][:, None] * d_out[pt[live]]).astype(np.float32))
    d_router = np.zeros(T * k, np.float32)
    d_router[dr[live]] = (d_out[pt[live]].astype(np.float64) * fwd["combine"][dr[live]].astype(np.float64)).sum(axis=1)
    hidden = ctx["hidden"]
    d_hidden = np.zeros((total, I), np.float32)
    d_w_down = np.zeros((E, H, I), np.float32)
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi > lo:
            d_hidden[lo:hi] = mxfp8.bf16_round(_mm(dy[lo:hi], w_down[e].T))                 # [rows, H] x [I, H]^T
            d_w_down[e] = mxfp8.bf16_round(_mm(dy[lo:hi].T, hidden[lo:hi].T))               # [H, rows] x [I, rows]^T
    g, u = ctx["gate"], ctx["up"]
    g_open, u_open = np.ones_like(g, dtype=bool), np.ones_like(u, dtype=bool)
    if limit > 0:
        lim = np.float32(limit)
        g_open, u_open = g < lim, (u > -lim) & (u < lim)
        g, u = np.minimum(g, lim), np.clip(u, -lim, lim)
    sg = (np.float32(1.0) / (np.float32(1.0) + np.exp(-g))).astype(np.float32)
    d_up = np.where(u_open, d_hidden * (g * sg), np.float32(0.0))
    d_gate = np.where(g_open, d_hidden * u * sg * (np.float32(1.0) + g * (np.float32(1.0) - sg)), np.float32(0.0))
    dgu = mxfp8.bf16_round(np.concatenate([d_gate, d_up], axis=1).astype(np.float32))
    rows = np.zeros((total, H), np.float32)
    rows[live] = x[pt[live]]
    d_x_buf = np.zeros((T * k, H), np.float32)
    d_w_cat = np.zeros((E, 2 * I, H), np.float32)
    for e in range(E):
        lo, hi = int(off[e]), int(off[e + 1])
        if hi > lo:
            dxr = mxfp8.bf16_round(_mm(dgu[lo:hi], np.concatenate([w_gate[e], w_up[e]]).T))   # [rows, 2I] x [H, 2I]^T
            sel = pr[lo:hi] >= 0
            d_x_buf[dr[lo:hi][sel]] = dxr[sel]
            d_w_cat[e] = mxfp8.bf16_round(_mm(dgu[lo:hi].T, rows[lo:hi].T))                   # [2I, rows] x [H, rows]^T
    d_x = fwd_epilogue(d_x_buf, np.ones((T, k), np.float32))
    return dict(d_x=d_x, d_router_weights=d_router.reshape(T, k), d_w_routed_gate=d_w_cat[:, :I], d_w_routed_up=d_w_cat[:, I:],
                d_w_routed_down=d_w_down, d_hidden=d_hidden, d_gate_up=dgu, d_y=dy)
