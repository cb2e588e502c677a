"""GPU parity of the MXFP8 MoE backward pass (CTA-pair GEMM variant) against the CPU oracle, which
itself agrees with autograd on the unquantised FFN to within MXFP8 noise (~7 %)."""
import numpy as np
import pytest
import torch

from oracle import moe as omoe

pytestmark = pytest.mark.gpu


def _f(t):
    return t.detach().float().cpu().numpy()


@pytest.mark.parametrize("shape_args,generation", [(("bwd-small", 4, 256, 256, 2, 384), 1), (("bwd-empty", 8, 512, 256, 2, 300), 3),
                                                   (("bwd-mid", 8, 1024, 512, 4, 512), 2)])
def test_backward_vs_oracle(native_lib, shape_args, generation):
    _forward_backward_vs_oracle(shape_args, generation, 0.0)


def test_clamped_activation_vs_oracle(native_lib):
    """The clamped-SwiGLU variant (the reference's c1 cells, campaigns/mok/README.md:82-84), with a
    bound low enough that a good share of gate and up values reach it."""
    from pipelink_b200 import _lib
    try:
        _forward_backward_vs_oracle(("bwd-clamp", 8, 512, 256, 2, 384), 2, 0.5)
    finally:
        _lib.call("plb_moe_set_swiglu_limit", 0.0)
    assert _lib.load().plb_moe_swiglu_limit() == 0.0


def _forward_backward_vs_oracle(shape_args, generation, limit):
    from pipelink_b200 import mok
    shape = mok.Shape(*shape_args)
    torch.manual_seed(5)
    E, H, I = shape.experts, shape.hidden, shape.intermediate
    wg = (torch.randn(E, I, H, device="cuda") * 0.05).to(torch.bfloat16)
    wu = (torch.randn(E, I, H, device="cuda") * 0.05).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device="cuda") * 0.05).to(torch.bfloat16)
    inputs = mok.MoKHost.new_inputs(shape, generation, "cuda")
    d_out = torch.randn(shape.tokens, H, device="cuda").to(torch.bfloat16)
    host = mok.MoKHost(shape, swiglu_limit=limit)
    host.load_weights(wg, wu, wd, train=True)
    fwd_plain = host.forward(inputs)["output"].clone()
    fwd_train = host.forward(inputs, train=True)["output"].clone()
    assert torch.equal(fwd_plain.view(torch.int16), fwd_train.view(torch.int16)), "the saving epilogue must not change the forward result"
    grads = host.backward(d_out)
    torch.cuda.synchronize()

    weights = omoe.quantize_weights(_f(wg), _f(wu), _f(wd))
    ctx = {}
    ref_f = omoe.forward_single_rank(_f(inputs.x), inputs.experts.cpu().numpy().astype(np.int32), inputs.router.cpu().numpy(),
                                     weights, padding=host.padding, capacity=host.capacity, context=ctx, limit=limit)
    ref = omoe.backward_single_rank(_f(inputs.x), inputs.router.cpu().numpy(), _f(wg), _f(wu), _f(wd), ref_f, ctx, _f(d_out),
                                    limit=limit)
    total = int(ref_f["schedule"]["num_tokens"][0])
    st = omoe.error_stats(ref_f["output"], _f(fwd_train))
    assert st["relative"] <= 2e-2, ("output", st)
    if limit > 0:
        live = ref_f["schedule"]["peer_rank"][:total] >= 0
        share = float((ctx["gate"][live] >= limit).mean()), float((np.abs(ctx["up"][live]) >= limit).mean())
        assert min(share) > 0.05, share                 # the bound is exercised on both operands
        closed = ctx["gate"][live] >= limit * 1.15      # beyond the bound by more than an E4M3 rounding step
        assert not _f(host.buffers["d_gate_up_routed"][:total])[live][:, :I][closed].any()
    # stage by stage: the combine backward is exact arithmetic on identical inputs up to the forward's y
    s = omoe.error_stats(ref["d_y"], _f(host.buffers["d_y_routed"])[:total])
    assert s["abs_max"] == 0.0, s
    for name, got, tol in (("d_hidden", host.buffers["d_hidden_routed"][:total], 3e-2),
                           ("d_gate_up", host.buffers["d_gate_up_routed"][:total], 4e-2),
                           ("d_router_weights", grads["d_router_weights"], 3e-2), ("d_x", grads["d_x"], 5e-2),
                           ("d_w_routed_down", grads["d_w_routed_down"], 5e-2), ("d_w_routed_gate", grads["d_w_routed_gate"], 5e-2),
                           ("d_w_routed_up", grads["d_w_routed_up"], 5e-2)):
        g = _f(got)
        assert np.isfinite(g).all(), name
        st = omoe.error_stats(ref[name], g)
        assert st["relative"] <= tol, (name, st)
    # experts that received no rows get exactly zero weight gradients
    empty = np.nonzero(ref_f["schedule"]["tokens_per_expert"] == 0)[0]
    for e in empty:
        assert not _f(grads["d_w_routed_down"][e]).any() and not _f(grads["d_w_routed_gate"][e]).any()


def test_recompute_pass_gives_the_same_gradients(native_lib):
    """A plain forward followed by backward(recompute=True) equals forward(train=True) + backward bit
    for bit: the recompute pass regenerates exactly the saved activations."""
    from pipelink_b200 import mok
    shape = mok.Shape("rec", 8, 512, 256, 2, 384)
    torch.manual_seed(9)
    E, H, I = shape.experts, shape.hidden, shape.intermediate
    mk = lambda *s: (torch.randn(*s, device="cuda") * 0.05).to(torch.bfloat16)
    host = mok.MoKHost(shape)
    host.load_weights(mk(E, I, H), mk(E, I, H), mk(E, H, I), train=True)
    inputs = mok.MoKHost.new_inputs(shape, 2, "cuda")
    d_out = torch.randn(shape.tokens, H, device="cuda").to(torch.bfloat16)
    host.forward(inputs, train=True)
    want = {k: v.clone() for k, v in host.backward(d_out).items()}
    for name in ("gate_routed_fp8", "up_routed_fp8", "hidden_routed_bf16"):
        host.buffers[name].zero_()                      # nothing may survive from the training forward
    host.forward(inputs)
    got = host.backward(d_out, recompute=True)
    for name, w in want.items():
        g = got[name]
        view = torch.int16 if g.dtype == torch.bfloat16 else torch.int32
        assert torch.equal(g.contiguous().view(view), w.contiguous().view(view)), name


@pytest.mark.parametrize("shape_args,generation,limit", [(("bf-small", 4, 256, 256, 2, 384), 1, 0.0), (("bf-empty", 8, 512, 256, 2, 300), 3, 0.0),
                                                         (("bf-mid", 8, 1024, 512, 4, 512), 2, 0.0), (("bf-clamp", 8, 512, 256, 2, 384), 2, 0.5)])
def test_bf16_precision_backward_vs_oracle(native_lib, shape_args, generation, limit):
    """The backward cells of the bf16 routed precision (campaigns/mok/README.md:86-104): no quantisation
    anywhere, so the device and the oracle differ only in fp32 summation order and one bf16 rounding
    per stored tensor: relative (sum|err| / sum|ref|) <= 1e-2 on every gradient, d_y exact."""
    from pipelink_b200 import _lib, mok
    shape = mok.Shape(*shape_args)
    torch.manual_seed(6)
    E, H, I = shape.experts, shape.hidden, shape.intermediate
    mk = lambda *s: (torch.randn(*s, device="cuda") * 0.05).to(torch.bfloat16)
    wg, wu, wd = mk(E, I, H), mk(E, I, H), mk(E, H, I)
    inputs = mok.MoKHost.new_inputs(shape, generation, "cuda")
    d_out = torch.randn(shape.tokens, H, device="cuda").to(torch.bfloat16)
    try:
        host = mok.MoKHost(shape, precision="bf16", swiglu_limit=limit)
        host.load_weights(wg, wu, wd, train=True)
        fwd_plain = host.forward(inputs)["output"].clone()
        fwd_train = host.forward(inputs, train=True)["output"].clone()
        assert torch.equal(fwd_plain.view(torch.int16), fwd_train.view(torch.int16))
        grads = {k: v.clone() for k, v in host.backward(d_out).items()}
        torch.cuda.synchronize()
        ctx = {}
        ref_f = omoe.forward_single_rank_bf16(_f(inputs.x), inputs.experts.cpu().numpy().astype(np.int32), inputs.router.cpu().numpy(),
                                              _f(wg), _f(wu), _f(wd), padding=host.padding, capacity=host.capacity, limit=limit,
                                              context=ctx)
        ref = omoe.backward_single_rank_bf16(_f(inputs.x), inputs.router.cpu().numpy(), _f(wg), _f(wu), _f(wd), ref_f, ctx, _f(d_out),
                                             limit=limit)
        total = int(ref_f["schedule"]["num_tokens"][0])
        assert omoe.error_stats(ref_f["output"], _f(fwd_train))["relative"] <= 1e-2
        assert omoe.error_stats(ref["d_y"], _f(host.buffers["d_y_routed"])[:total])["abs_max"] == 0.0
        for name, got in (("d_hidden", host.buffers["d_hidden_routed"][:total]), ("d_gate_up", host.buffers["d_gate_up_routed"][:total]),
                          ("d_router_weights", grads["d_router_weights"]), ("d_x", grads["d_x"]),
                          ("d_w_routed_down", grads["d_w_routed_down"]), ("d_w_routed_gate", grads["d_w_routed_gate"]),
                          ("d_w_routed_up", grads["d_w_routed_up"])):
            g = _f(got)
            assert np.isfinite(g).all(), name
            st = omoe.error_stats(ref[name], g)
            assert st["relative"] <= 1e-2, (name, st)
        for e in np.nonzero(ref_f["schedule"]["tokens_per_expert"] == 0)[0]:
            assert not _f(grads["d_w_routed_down"][e]).any() and not _f(grads["d_w_routed_gate"][e]).any()
        # the recompute cell: a plain forward, then the activations regenerated inside the backward pass
        for name in ("gate_routed_bf16", "up_routed_bf16"):
            host.buffers[name].zero_()
        host.forward(inputs)
        again = host.backward(d_out, recompute=True)
        for name, w in grads.items():
            g = again[name]
            view = torch.int16 if g.dtype == torch.bfloat16 else torch.int32
            assert torch.equal(g.contiguous().view(view), w.contiguous().view(view)), ("recompute", name)
    finally:
        _lib.call("plb_moe_set_swiglu_limit", 0.0)
