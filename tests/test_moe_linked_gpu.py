"""The MoE grouped GEMMs as linked images (stages/moe packed separately, joined by the link
driver) against the library's own kernels: same inputs, same bits, for the gate/up projection
(rows in place, and rows pulled by the comm owner inside the image) and the down projection, as two
launches and as the one-launch forward image."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def linked_dir(native_lib):
    from pipelink_b200 import moe_linked
    return moe_linked.ensure_built()


@pytest.mark.parametrize("shape_args,generation", [(("lk-small", 4, 256, 256, 2, 384), 1), (("lk-empty", 8, 512, 256, 2, 300), 3),
                                                   (("lk-wide", 8, 4096, 512, 4, 1024), 2)])
def test_linked_images_equal_the_library_kernels(linked_dir, shape_args, generation):
    from pipelink_b200 import mok, moe_linked
    shape = mok.Shape(*shape_args)
    torch.manual_seed(5)
    E, H, I = shape.experts, shape.hidden, shape.intermediate
    mk = lambda *s: (torch.randn(*s, device="cuda") * 0.05).to(torch.bfloat16)
    wg, wu, wd = mk(E, I, H), mk(E, I, H), mk(E, H, I)
    lib, lnk = mok.MoKHost(shape), mok.MoKHost(shape)
    for h in (lib, lnk):
        h.load_weights(wg, wu, wd)
    linked = moe_linked.LinkedMoE(lnk, linked_dir)
    try:
        for step in range(2):
            inputs = mok.MoKHost.new_inputs(shape, generation + step, "cuda")
            want = lib.forward(inputs)
            for dispatch, one_launch in ((False, False), (True, False), (False, True), (True, True), (False, "full"), (True, "full")):
                lnk.status.reset()
                lnk.fused_dispatch = dispatch               # quantise_tokens then also writes the scale rows
                for name in ("x_routed_fp8", "hidden_routed_fp8"):
                    lnk.buffers[name].fill_(77)
                lnk.buffers["combine_buffer"].fill_(float("nan"))
                lnk.schedule_into(inputs.experts[None])
                lnk.x_buffer.copy_(inputs.x)
                lnk.router_weight_buffer.copy_(inputs.router)
                lnk.dispatch()                              # with dispatch: quantise only, the image pulls
                if one_launch == "full":                    # ... and the weighted epilogue in the same launch
                    lnk.buffers["output"].fill_(float("nan"))
                    out = linked.forward_full(dispatch=dispatch)
                elif one_launch:                            # both projections in one launch of the fwd image
                    linked.forward_ffn(dispatch=dispatch)
                    out = lnk.fwd_epilogue()
                else:
                    linked.gemm_gate_up(dispatch=dispatch)
                    linked.gemm_down()
                    out = lnk.fwd_epilogue()
                torch.cuda.synchronize()
                lnk.status.check("linked forward")
                total = int(lib.schedule.num_tokens.item())
                tag = (step, "dispatch" if dispatch else "in place", "one launch" if one_launch else "two launches")
                assert torch.equal(lnk.buffers["x_routed_fp8"][:total], want["x_routed_data"][:total]), tag
                assert torch.equal(lnk.buffers["hidden_routed_fp8"][:total], want["hidden_routed_data"][:total]), tag
                assert torch.equal(lnk.buffers["hidden_routed_sc"][: total // 128], want["hidden_routed_scale"][: total // 128]), tag
                live = lib.schedule.dest_row[:total] >= 0
                rows = lib.schedule.dest_row[:total][live].long()
                assert torch.equal(lnk.buffers["combine_buffer"][rows].view(torch.int16), want["combine_buffer"][rows].view(torch.int16)), tag
                assert torch.equal(out.view(torch.int16), want["output"].view(torch.int16)), tag
    finally:
        linked.close()


def test_linked_image_refuses_a_bad_schedule(linked_dir):
    """The linked owners make the same check as the library kernel: a row count off the 256-row
    grid is reported through the status record and nothing is written."""
    from pipelink_b200 import mok, moe_linked
    shape = mok.Shape("lk-bad", 4, 256, 256, 1, 512)
    host = mok.MoKHost(shape)
    mk = lambda *s: (torch.randn(*s, device="cuda") * 0.05).to(torch.bfloat16)
    host.load_weights(mk(4, 256, 256), mk(4, 256, 256), mk(4, 256, 256))
    inputs = mok.MoKHost.new_inputs(shape, 1, "cuda")
    host.forward(inputs)
    linked = moe_linked.LinkedMoE(host, linked_dir)
    try:
        host.schedule.num_tokens.fill_(384)
        host.buffers["hidden_routed_fp8"].fill_(77)
        linked.gemm_gate_up()
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="status 6"):
            host.status.check("linked gate/up on a bad schedule")
        assert (host.buffers["hidden_routed_fp8"] == 77).all()
    finally:
        linked.close()
