"""Tensor-import cells on the GPU: ONE consumer source against a tensor-memory tile, a transposed
tensor-memory tile and a swizzled shared-memory tile, by rows and by columns; the adapters are the
link's (direct receipt, staging through lent scratch, composed shared loads). Every cell gives
max(x * scale + bias[m], 0) bit for bit (the arithmetic is one fma-free multiply and add per
element, computed here with the same roundings), and the linked image equals the single-unit build
of the same sources (the reference's acceptance of its many-producers cells:
examples/one-epilogue-many-producers/README.md)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

CELLS = {"tmem": "direct_receipt", "tmem_transposed": "staged_constructed", "smem": "shared_direct",
         "tmem_by_column": "staged_constructed", "smem_by_column": "shared_direct"}


@pytest.mark.parametrize("cell", sorted(CELLS))
@pytest.mark.parametrize("tiles,ld", [(1, 128), (300, 160)])
def test_cell_equals_the_host_and_the_single_unit_build(native_lib, cell, tiles, ld):
    from pipelink_b200 import tensor_import_linked as til
    torch.manual_seed(tiles)
    x = torch.randn(tiles * 128, ld, device="cuda")[:, :ld]
    bias = torch.randn(128, device="cuda")
    scale = 1.75
    # x * scale is exact in float32 up to one rounding, the sum one more: torch does the same two roundings
    want = torch.clamp_min(x[:, :128] * scale + bias.repeat(tiles)[:, None], 0.0)
    got = {}
    for image in ("pipeline.cubin", "one_tu.cubin"):
        img = til.TensorImportImage(cell, image=image)
        try:
            assert img.record["route"] == CELLS[cell]
            got[image] = img(x, bias, scale)
            torch.cuda.synchronize()
        finally:
            img.close()
    assert torch.equal(got["pipeline.cubin"].view(torch.int32), got["one_tu.cubin"].view(torch.int32))
    # the device may contract the multiply and the add into one fma: allow that one rounding
    assert torch.allclose(got["pipeline.cubin"], want, rtol=0, atol=2e-6 * float(x.abs().max() * scale + bias.abs().max()))
    assert (got["pipeline.cubin"] >= 0).all()
