"""Causal prefill attention as linked images (stages/attention: load, MMA, gather and softmax owners
packed separately, joined by the link driver) against the library kernel: same inputs, same bits
for O and LSE, plain, with a sliding window, and with the soft cap that only the image holding the
softcap owner applies; the single-unit build of the same stage sources too."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def images(native_lib):
    from pipelink_b200 import attention_linked
    attention_linked.ensure_built()
    linked, control = attention_linked.LinkedAttention(), attention_linked.LinkedAttention(image="one_tu.cubin")
    yield linked, control
    linked.close()
    control.close()


@pytest.mark.parametrize("B,S,Hq,Hkv,window,softcap", [(1, 1024, 8, 2, 0, 0.0), (2, 512, 4, 2, 0, 0.0), (1, 2048, 8, 4, 384, 0.0),
                                                       (1, 1024, 4, 1, 0, 30.0), (1, 1536, 8, 2, 512, 20.0)])
def test_linked_attention_equals_the_library_kernel(images, B, S, Hq, Hkv, window, softcap):
    from pipelink_b200 import attention
    g = torch.Generator(device="cuda").manual_seed(7 + S + Hq)
    mk = lambda h: (torch.randn(B, S, h, 128, generator=g, device="cuda") * 0.8).to(torch.bfloat16)
    q, k, v = mk(Hq), mk(Hkv), mk(Hkv)
    want_o, want_lse = attention.attention_fwd(q, k, v, window=window, softcap=softcap)
    for arm, tag in zip(images, ("linked", "single unit")):
        o, lse = arm.forward(q, k, v, window=window, softcap=softcap)
        torch.cuda.synchronize()
        assert torch.equal(o.view(torch.int16), want_o.view(torch.int16)), tag
        assert torch.equal(lse.view(torch.int32), want_lse.view(torch.int32)), tag
    if softcap > 0:
        # the variant is in the image, not in a flag: the plain composition ignores the cap
        plain_o, _ = attention.attention_fwd(q, k, v, window=window)
        assert not torch.equal(plain_o.view(torch.int16), want_o.view(torch.int16))


def test_linked_attention_wants_head_pairs(images):
    q = torch.zeros(1, 128, 3, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.zeros(1, 128, 3, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="head-pair"):
        images[0].forward(q, k, k)


def test_linked_context_parallel_image_on_a_group_of_one(images):
    """The `prefill_cp` composition (load owner behind readiness counters + the gather owner's ticketed
    K/V push) on one rank: the gather warps move this rank's K/V from its local tensors into its own
    gathered buffers while the load owner waits for the counts; the plain kernel's bits, three steps."""
    from pipelink_b200 import _lib, attention as att, ep
    S, Hq, Hkv = 2048, 8, 2
    g = torch.Generator(device="cuda").manual_seed(99)
    mk = lambda h: (torch.randn(S, h, 128, generator=g, device="cuda") * 0.8).to(torch.bfloat16)
    q, k, v = mk(Hq), mk(Hkv), mk(Hkv)
    want_o, want_lse = att.attention_fwd(q[None], k[None], v[None])
    layout = att.CpRank.slab_layout(S, Hkv)
    slab = ep.sym_alloc(layout["nbytes"])
    try:
        rnk = att.CpRank(S, Hq, Hkv, 0, 1, [slab], layout, "cuda", fused_push=True)
        rnk.k_gather.fill_(float("nan"))
        rnk.v_gather.fill_(float("nan"))
        for step in range(3):
            o, lse = images[0].attend_and_push(rnk, q, k, v)
            torch.cuda.synchronize()
            rnk.status.check(f"linked context-parallel image, step {step}")
            assert torch.equal(o.view(torch.int16), want_o[0].view(torch.int16)), step
            assert torch.equal(lse, want_lse), step
            assert (rnk.ready.cpu().numpy() == (step + 1) * att.CpRank.PARTS).all()
    finally:
        torch.cuda.synchronize()
        _lib.call("plb_sym_free", slab)
