"""The MoE oracle against autograd: its forward and backward passes restate the reference's
quantisation points, so they must agree with the unquantised fp64 FFN to within MXFP8 noise, with
and without the clamped activation (campaigns/mok/README.md:82-84: the c0 / c1 cells)."""
import numpy as np
import pytest
import torch

from oracle import moe as omoe
from oracle import mxfp8


def _rel(ref, got):
    ref, got = np.asarray(ref, np.float64), np.asarray(got, np.float64)
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))


@pytest.mark.parametrize("limit", [0.0, 1.0])
def test_activation_matches_autograd(limit):
    rng = np.random.default_rng(3)
    g = (rng.standard_normal((64, 32)) * 2).astype(np.float32)
    u = (rng.standard_normal((64, 32)) * 2).astype(np.float32)
    gt, ut = torch.tensor(g, dtype=torch.float64), torch.tensor(u, dtype=torch.float64)
    if limit > 0:
        want = torch.nn.functional.silu(torch.clamp(gt, max=limit)) * torch.clamp(ut, -limit, limit)
    else:
        want = torch.nn.functional.silu(gt) * ut
    assert np.allclose(omoe.silu_mul(g, u, limit), want.numpy(), rtol=1e-5, atol=1e-6)
    if limit > 0:
        assert (g >= limit).mean() > 0.1 and (np.abs(u) >= limit).mean() > 0.1


def _dense_ffn(x, routes, router_w, wg, wu, wd, limit):
    """fp64 autograd model of the routed FFN: out[t] = sum_s w[t, s] * down_e(act(gate_e x, up_e x))."""
    T, k = routes.shape
    out = torch.zeros(T, x.shape[1], dtype=torch.float64)
    for s in range(k):
        for e in range(wg.shape[0]):
            sel = torch.nonzero(torch.from_numpy(routes[:, s] == e)).flatten()
            if sel.numel() == 0:
                continue
            g, u = x[sel] @ wg[e].T, x[sel] @ wu[e].T
            if limit > 0:
                g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
            y = (torch.nn.functional.silu(g) * u) @ wd[e].T
            out = out.index_add(0, sel, router_w[sel, s:s + 1] * y)
    return out


@pytest.mark.parametrize("limit", [0.0, 0.5])
def test_forward_backward_match_autograd_within_mxfp8_noise(limit):
    rng = np.random.default_rng(11)
    E, H, I, k, T = 4, 256, 128, 2, 96
    bf = lambda a: mxfp8.bf16_round(a.astype(np.float32))
    wg, wu = bf(rng.standard_normal((E, I, H)) * 0.05), bf(rng.standard_normal((E, I, H)) * 0.05)
    wd = bf(rng.standard_normal((E, H, I)) * 0.05)
    x, d_out = bf(rng.standard_normal((T, H))), bf(rng.standard_normal((T, H)))
    routes = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    router_w = rng.random((T, k)).astype(np.float32)
    router_w /= router_w.sum(axis=1, keepdims=True)

    ctx = {}
    weights = omoe.quantize_weights(wg, wu, wd)
    fwd = omoe.forward_single_rank(x, routes, router_w, weights, context=ctx, limit=limit)
    bwd = omoe.backward_single_rank(x, router_w, wg, wu, wd, fwd, ctx, d_out, limit=limit)

    t = lambda a: torch.tensor(a, dtype=torch.float64, requires_grad=True)
    xt, rt, wgt, wut, wdt = t(x), t(router_w), t(wg), t(wu), t(wd)
    out = _dense_ffn(xt, routes, rt, wgt, wut, wdt, limit)
    out.backward(torch.tensor(d_out, dtype=torch.float64))
    assert _rel(out.detach().numpy(), fwd["output"]) < 0.08
    for name, ref in (("d_x", xt.grad), ("d_router_weights", rt.grad), ("d_w_routed_gate", wgt.grad),
                      ("d_w_routed_up", wut.grad), ("d_w_routed_down", wdt.grad)):
        # a bound decided on MXFP8-rounded gate / up flips for elements within the rounding step of
        # it, which adds noise to the gradients that pass the activation; the decision itself is
        # checked exactly below
        tol = 0.10 if limit == 0 or name in ("d_router_weights", "d_w_routed_down") else 0.30
        assert _rel(ref.numpy(), bwd[name]) < tol, (name, _rel(ref.numpy(), bwd[name]))
    # the activation's backward on the oracle's own operands: exact up to the bf16 rounding of the result
    gq = torch.tensor(mxfp8.dequantize(*mxfp8.quantize(ctx["gate"])), dtype=torch.float64, requires_grad=True)
    uq = torch.tensor(mxfp8.dequantize(*mxfp8.quantize(ctx["up"])), dtype=torch.float64, requires_grad=True)
    gc, uc = (torch.clamp(gq, max=limit), torch.clamp(uq, -limit, limit)) if limit > 0 else (gq, uq)
    (torch.nn.functional.silu(gc) * uc).backward(torch.tensor(bwd["d_hidden"], dtype=torch.float64))
    want = torch.cat([gq.grad, uq.grad], dim=1).numpy()
    if limit > 0:
        # torch.clamp passes the gradient at equality; the reference and the oracle do not
        at = np.concatenate([gq.detach().numpy() == limit, np.abs(uq.detach().numpy()) == limit], axis=1)
        want[at] = 0.0
    assert _rel(want, bwd["d_gate_up"]) < 5e-3
    assert ((want == 0) == (bwd["d_gate_up"] == 0)).mean() > 0.999
    if limit > 0:
        live = fwd["schedule"]["peer_rank"][:int(fwd["schedule"]["num_tokens"][0])] >= 0
        assert (ctx["gate"][live] >= limit).mean() > 0.05
        plain = omoe.forward_single_rank(x, routes, router_w, weights)["output"]
        assert _rel(plain, fwd["output"]) > 0.05          # the bound changes the result


@pytest.mark.parametrize("limit", [0.0, 0.5])
def test_bf16_precision_forward_matches_dense_model(limit):
    """The bf16 routed precision has no quantisation noise: only bf16 roundings separate it from fp64."""
    rng = np.random.default_rng(12)
    E, H, I, k, T = 4, 256, 128, 2, 96
    bf = lambda a: mxfp8.bf16_round(a.astype(np.float32))
    wg, wu = bf(rng.standard_normal((E, I, H)) * 0.05), bf(rng.standard_normal((E, I, H)) * 0.05)
    wd, x = bf(rng.standard_normal((E, H, I)) * 0.05), bf(rng.standard_normal((T, H)))
    routes = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    router_w = rng.random((T, k)).astype(np.float32)
    got = omoe.forward_single_rank_bf16(x, routes, router_w, wg, wu, wd, limit=limit)
    t = lambda a: torch.tensor(a, dtype=torch.float64)
    want = _dense_ffn(t(x), routes, t(router_w), t(wg), t(wu), t(wd), limit)
    assert _rel(want.numpy(), got["output"]) < 6e-3


def test_spot_rows_equal_rows_of_the_full_forward():
    """forward_token_rows (what the full-size GPU test is held to) against forward_single_rank on a
    problem small enough to run whole: the sampled tokens' outputs are the same bits."""
    from oracle import routing as oroute
    rng = np.random.default_rng(1)
    E, H, I, T, k = 8, 256, 256, 300, 2
    w = [mxfp8.bf16_round(rng.standard_normal(s, dtype=np.float32) * np.float32(0.05))
         for s in ((E, I, H), (E, I, H), (E, H, I))]
    weights = omoe.quantize_weights(*w)
    x = mxfp8.bf16_round(rng.standard_normal((T, H), dtype=np.float32))
    ids, rw = oroute.route_topk(rng.standard_normal((T, E), dtype=np.float32), k)
    full = omoe.forward_single_rank(x, ids, rw, weights)["output"]

    def expert_weights(e):
        out = []
        for name, (R, C) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
            q, sc = weights[name]
            out.append((q[e], mxfp8.pack_scales(mxfp8.unpack_scales(sc, E * R, C)[e * R:(e + 1) * R])))
        return out

    sel = np.array([0, 5, 17, 123, 299])
    got = omoe.forward_token_rows(x[sel], ids[sel], rw[sel], expert_weights)
    assert np.array_equal(got, full[sel])


@pytest.mark.parametrize("limit", [0.0, 0.75])
def test_bf16_backward_oracle_matches_autograd(limit):
    """backward_single_rank_bf16 against fp64 autograd of the unquantised FFN: with no quantisation on
    the path only bf16 roundings separate them (the MXFP8 oracle needs a few per cent)."""
    from oracle import routing as oroute
    rng = np.random.default_rng(4)
    E, H, I, T, k = 4, 128, 128, 96, 2
    bf = mxfp8.bf16_round
    wg, wu, wd = (bf(rng.standard_normal(s, dtype=np.float32) * np.float32(0.2)) for s in ((E, I, H), (E, I, H), (E, H, I)))
    x = bf(rng.standard_normal((T, H), dtype=np.float32))
    d_out = bf(rng.standard_normal((T, H), dtype=np.float32))
    ids, rw = oroute.route_topk(rng.standard_normal((T, E), dtype=np.float32), k)
    ctx = {}
    fwd = omoe.forward_single_rank_bf16(x, ids, rw, wg, wu, wd, limit=limit, context=ctx)
    got = omoe.backward_single_rank_bf16(x, rw, wg, wu, wd, fwd, ctx, d_out, limit=limit)
    t = lambda a: torch.tensor(a, dtype=torch.float64, requires_grad=True)
    xt, rwt, wgt, wut, wdt = t(x), t(rw), t(wg), t(wu), t(wd)
    out = _dense_ffn(xt, ids, rwt, wgt, wut, wdt, limit)
    out.backward(torch.tensor(d_out, dtype=torch.float64))
    assert _rel(out.detach().numpy(), fwd["output"]) < 1e-2
    # with a bound, the decision is taken on bf16-rounded gate / up: an element within half a bf16 step
    # of the bound flips, and each flip is a whole gradient term (the MXFP8 test above carries the same note)
    tol = 1e-2 if limit == 0 else 8e-2
    for name, ref in (("d_x", xt.grad), ("d_router_weights", rwt.grad), ("d_w_routed_gate", wgt.grad),
                      ("d_w_routed_up", wut.grad), ("d_w_routed_down", wdt.grad)):
        assert _rel(ref.numpy(), got[name]) < tol, name
