"""The MXFP8 oracle against independent implementations available on the CPU:
torch's float8_e4m3fn / float8_e8m0fnu casts and exact integer reasoning about the rule."""
import numpy as np
import torch

from oracle import mxfp8


def test_e4m3_encode_matches_torch_cast():
    rng = np.random.default_rng(0)
    parts = [rng.standard_normal(50000).astype(np.float32) * s for s in (1e-3, 1e-2, 0.1, 1, 10, 100, 300)]
    edge = np.array([0, -0.0, 448, 449, 463.9, 464, 464.1, 480, 1e9, -1e9, 2**-9, 2**-10, 2**-10 * 1.0001,
                     2**-6, 0.0175, 3 * 2**-10, 5 * 2**-10], dtype=np.float32)
    x = np.concatenate(parts + [edge])
    mine = mxfp8.float_to_e4m3(x)
    ref = torch.from_numpy(np.clip(x, -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(mine, ref)


def test_e4m3_decode_matches_torch():
    b = np.arange(256, dtype=np.uint8)
    mine = mxfp8.e4m3_to_float(b)
    ref = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.isnan(mine), np.isnan(ref))
    assert np.array_equal(mine[~np.isnan(mine)], ref[~np.isnan(ref)])


def test_e8m0_decode_matches_torch():
    b = np.arange(255, dtype=np.uint8)
    ref = torch.arange(255, dtype=torch.uint8).view(torch.float8_e8m0fnu).float().numpy()
    assert np.array_equal(mxfp8.e8m0_value(b), ref)


def test_scale_rule_is_exact_ceil_log2():
    # powers of two times 448 land exactly; one ulp above moves to the next exponent
    for n in (-20, -1, 0, 1, 7, 30):
        a = np.float32(448.0 * 2.0**n)
        assert int(mxfp8.e8m0_from_amax(a)) - 127 == n
        assert int(mxfp8.e8m0_from_amax(np.nextafter(a, np.float32(np.inf)))) - 127 == n + 1
        assert int(mxfp8.e8m0_from_amax(np.nextafter(a, np.float32(0)))) - 127 == n
    assert int(mxfp8.e8m0_from_amax(np.float32(0))) == 0
    assert int(mxfp8.e8m0_from_amax(np.float32(1e-45))) == 0
    # never saturates: amax * 2^-e <= 448
    rng = np.random.default_rng(1)
    a = np.abs(rng.standard_normal(100000).astype(np.float32)) * np.float32(10.0) ** rng.integers(-8, 8, 100000)
    e = mxfp8.e8m0_from_amax(a)
    scaled = a.astype(np.float64) * np.ldexp(1.0, 127 - e.astype(np.int64))
    assert (scaled <= 448.0).all() and (scaled > 224.0 - 1e-9).all()


def test_scale_layout_is_the_reference_tile_layout():
    rows, cols = 256, 384
    off = mxfp8.scale_offsets(rows, cols)
    assert sorted(off.reshape(-1)) == list(range(rows * cols // 32))
    r, g = 130, 9  # block (1, 2), row 2 of the block, group 1
    assert off[r, g] == (1 * 3 + 2) * 512 + (2 % 32) * 16 + (2 // 32) * 4 + 1
    r, g = 100, 3
    assert off[r, g] == 0 * 512 + (100 % 32) * 16 + (100 // 32) * 4 + 3
    sc = np.arange(rows * cols // 32, dtype=np.uint8).reshape(rows, cols // 32)
    assert np.array_equal(mxfp8.unpack_scales(mxfp8.pack_scales(sc), rows, cols), sc)


def test_quantize_roundtrip_properties():
    rng = np.random.default_rng(2)
    x = mxfp8.bf16_round(rng.standard_normal((256, 512)).astype(np.float32) * 3)
    x[5, 32:64] = 0.0          # an all-zero block
    x[7, 0] = 3.0e38           # a huge element
    q, sc = mxfp8.quantize(x)
    d = mxfp8.dequantize(q, sc)
    s = mxfp8.unpack_scales(sc, 256, 512)
    assert s[5, 1] == 0 and (q[5, 32:64] == 0).all()
    assert np.isfinite(d).all()
    blocks = x.reshape(256, 16, 32)
    amax = np.abs(blocks).max(axis=2)
    # error bound: half an E4M3 ulp at the top binade of the block (2^(e+8-3) / 2)
    bound = np.ldexp(1.0, s.astype(np.int64) - 127 + 8 - 4)
    assert (np.abs(d - x).reshape(256, 16, 32).max(axis=2) <= bound + 1e-30).all()
    assert (amax <= 448.0 * np.ldexp(1.0, s.astype(np.int64) - 127)).all()
    # idempotent in value: every dequantised number is exactly representable again
    q2, sc2 = mxfp8.quantize(d)
    assert np.array_equal(mxfp8.dequantize(q2, sc2), d)
    # transposed orientation = quantise of the transpose
    qt, sct = mxfp8.quantize_transposed(x)
    assert qt.shape == (512, 256) and sct.shape == (4, 2, 32, 16)
