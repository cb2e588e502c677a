"""BASELINE config 0 on the GPU: the LTO-linked three-stage MXFP8 GEMM against the CPU oracle,
and the linked image against its same-source one-TU control (bitwise, the reference's own parity
criterion, examples/hopper-gemm-split/run.py)."""
import numpy as np
import pytest
import torch

from oracle import gemm3 as og

pytestmark = pytest.mark.gpu


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def images(native_lib):
    from pipelink_b200 import gemm3
    link_dir = gemm3.ensure_built()
    linked, control = gemm3.Gemm3(link_dir), gemm3.Gemm3(link_dir, "one_tu.cubin")
    yield linked, control
    linked.close()
    control.close()


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (1024, 1024, 1024)])
def test_linked_gemm_vs_oracle_and_one_tu(images, M, N, K):
    linked, control = images
    case = og.make_case(M, N, K, seed=0)
    dev = {k: _t(case[k]) for k in ("aq", "asc", "bq", "bsc")}
    bias = torch.from_numpy(case["bias"]).to(torch.bfloat16).cuda()
    outs = []
    for g in (linked, control):
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")   # poison
        g.run(dev["aq"], dev["asc"], dev["bq"], dev["bsc"], bias, out)
        torch.cuda.synchronize()
        outs.append(out)
    ref = og.expected(case)
    stats = og.compare(ref, outs[0].float().cpu().numpy())
    assert stats["violations"] == 0 and stats["rel_l2"] <= 1e-2, stats
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16)), "linked and one-TU images must agree bitwise"


def test_linked_vs_one_tu_latency(images):
    """Reports both latencies; the linked image must be within 3 % of the one-TU control
    (the reference's gate for linked/one-TU ratios, campaigns/mok/README.md:262-276)."""
    linked, control = images
    case = og.make_case(1024, 1024, 1024, seed=0)
    dev = {k: _t(case[k]) for k in ("aq", "asc", "bq", "bsc")}
    bias = torch.from_numpy(case["bias"]).to(torch.bfloat16).cuda()
    out = torch.empty((1024, 1024), dtype=torch.bfloat16, device="cuda")
    times = []
    for g in (linked, control):
        g.run(dev["aq"], dev["asc"], dev["bq"], dev["bsc"], bias, out)
        best = min(g.session.time((8, 8, 1), n=50) for _ in range(5))
        times.append(best)
    print(f"linked {times[0] * 1e3:.2f} us, one-TU {times[1] * 1e3:.2f} us, ratio {times[0] / times[1]:.4f}")
    assert times[0] <= times[1] * 1.03 + 0.002


@pytest.mark.parametrize("M,N,K", [(256, 384, 512), (1024, 1024, 1024)])
def test_hosted_open_equals_hostless_and_replays_from_a_graph(images, M, N, K):
    """The broker route: the group's provider is queried, builds the three parameter blocks (tensor
    maps included) and the launch must be bitwise the host-less one; one captured CUDA graph
    replays it onto fresh poison."""
    from pipelink_b200 import gemm3
    linked, _ = images
    case = og.make_case(M, N, K, seed=1)
    dev = {k: _t(case[k]) for k in ("aq", "asc", "bq", "bsc")}
    bias = torch.from_numpy(case["bias"]).to(torch.bfloat16).cuda()
    plain = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    linked.run(dev["aq"], dev["asc"], dev["bq"], dev["bsc"], bias, plain)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    hosted = gemm3.Gemm3Hosted(dev["aq"], dev["asc"], dev["bq"], dev["bsc"], bias, out)
    try:
        assert hosted.session.geometry[0] == (M // 128, N // 128, 1)
        assert [t["ring_depth"] for t in hosted.session.transfers] == [hosted.session.link["bindings"]["pipelink_gemm_depth"][0]] * 2
        hosted.run()
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), plain.view(torch.int16))
        graph = hosted.capture()
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), plain.view(torch.int16))
    finally:
        hosted.close()
