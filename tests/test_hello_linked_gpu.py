"""The hello image on the GPU: the caller's loop and the provider's function were packed apart and
meet through a generated trampoline; the result equals 2*x bit for bit, and equals the single-unit
build of the same two sources (the reference's acceptance of the same pair:
examples/hello-callable/README.md, "All three bitwise PASS")."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("count", [1, 127, 128 * 1024, 128 * 1024 * 3 + 5])
def test_linked_call_equals_the_host_and_the_single_unit_build(native_lib, count):
    from pipelink_b200 import hello_linked
    x = torch.randn(count, device="cuda")
    x[0] = float("inf")
    want = (x.cpu().numpy() * np.float32(2.0)).view(np.uint32)
    for image in ("pipeline.cubin", "one_tu.cubin"):
        img = hello_linked.HelloImage(image=image)
        try:
            out = torch.full((count + 4,), -7.0, device="cuda")
            img(x, out[:count])
            torch.cuda.synchronize()
            assert np.array_equal(out[:count].cpu().numpy().view(np.uint32), want), image
            assert (out[count:] == -7.0).all(), image      # nothing behind `count` is written
        finally:
            img.close()
