"""The decode interpreter as a linked image (stages/decode: the stream owner and the interpreter
owner packed separately, joined by the link driver) against the library's kernel: the same weights,
caches and start token give the same tokens, logits and KV rows, bit for bit; the single-unit build
of the same stage sources too; and the linked image reports a dependency that is never signalled
the way the library kernel does."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _weights(layers, vocab, seed=3):
    from pipelink_b200 import decode as hd
    torch.manual_seed(seed)
    mk = lambda *s: (torch.randn(*s, device="cuda") * 0.02).to(torch.bfloat16)
    return dict(qkv_w=mk(layers, hd.QKV_ROWS, hd.HIDDEN), o_w=mk(layers, hd.HIDDEN, hd.HIDDEN),
                up_w=mk(layers, hd.FFN, hd.HIDDEN), gate_w=mk(layers, hd.FFN, hd.HIDDEN), down_w=mk(layers, hd.HIDDEN, hd.FFN),
                attn_norm=(1 + 0.1 * torch.randn(layers, hd.HIDDEN, device="cuda")).to(torch.bfloat16),
                mlp_norm=(1 + 0.1 * torch.randn(layers, hd.HIDDEN, device="cuda")).to(torch.bfloat16),
                lm_norm=torch.ones(hd.HIDDEN, device="cuda", dtype=torch.bfloat16), lm_head=mk(vocab, hd.HIDDEN))


@pytest.mark.parametrize("layers,vocab,pos,steps", [(2, 4096, 0, 6), (3, 32000, 300, 5), (2, 8192, 1100, 4)])
def test_linked_decode_equals_the_library_kernel(native_lib, layers, vocab, pos, steps):
    from pipelink_b200 import decode as hd, decode_linked
    w = _weights(layers, vocab)
    sessions = [hd.DecodeSession(w, max_seq_len=pos + steps + 8) for _ in range(3)]
    prefix = torch.randn(layers, max(pos, 1), hd.KV_HEADS, hd.HEAD_DIM, device="cuda").to(torch.bfloat16)
    for s in sessions:
        if pos:
            s.k_cache[:, :pos].copy_(prefix[:, :pos])
            s.v_cache[:, :pos].copy_(prefix[:, :pos].flip(1))
        s.start(17, pos)
    lib, lnk, one = sessions
    lib.decode(steps)
    linked, control = decode_linked.LinkedDecode(lnk), decode_linked.LinkedDecode(one, image="one_tu.cubin")
    try:
        linked.decode(steps)
        control.decode(steps)
        torch.cuda.synchronize()
        for other, tag in ((lnk, "linked"), (one, "single unit")):
            assert torch.equal(other.token_out, lib.token_out), tag
            assert int(other.pos.item()) == pos + steps, tag
            assert torch.equal(other.logits.view(torch.int16), lib.logits.view(torch.int16)), tag
            assert torch.equal(other.k_cache.view(torch.int16), lib.k_cache.view(torch.int16)), tag
            assert torch.equal(other.v_cache.view(torch.int16), lib.v_cache.view(torch.int16)), tag
        assert (lib.token_out[pos + 1:pos + 1 + steps] >= 0).all()
    finally:
        linked.close()
        control.close()


def test_linked_decode_reports_a_dependency_that_never_comes(native_lib):
    """A wait that runs out in the linked image ends the launch with a status record; the context stays usable."""
    from pipelink_b200 import decode as hd, decode_linked
    w = _weights(1, 2048)
    s = hd.DecodeSession(w, max_seq_len=32)
    s.start(5, 0)
    linked = decode_linked.LinkedDecode(s)
    try:
        saved = s.instructions.clone()
        inst = s.instructions.view(s.num_sms, -1, 32)
        first = int((inst[0, :, 0] != 0).nonzero()[0])
        inst[:, first, 6] = 0            # every CTA's first instruction waits on counter 0 ...
        inst[:, first, 7] = 1 << 30      # ... for a count nothing will ever reach
        linked.step()
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="status"):
            s.status.check("linked decode with an unsignalled dependency")
        s.instructions.copy_(saved)
        s.start(5, 0)
        linked.decode(2)
        assert (s.token_out[1:3] >= 0).all()
    finally:
        linked.close()
