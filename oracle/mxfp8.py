"""CPU oracle for MXFP8 quantisation — TEST INFRASTRUCTURE, never on the product path.

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import this module.

PARITY UNPINNED for the scale rule: the reference's arithmetic
(``mxfp8::quantize_tile`` / ``quantize_single_block`` / ``ops.mxfp8_quantize``) lives in the
un-vendored submodule ``cursor/mixture-of-kittens`` @ f3a8bd2 (``csrc/mxfp8.cuh``) and is
absent from the reference tree; only its call sites and data layout are present
(campaigns/mok/port/act_gptoss/swiglu.cuh:187,349,367,395-409;
campaigns/mok/host/resources.py:62-77; campaigns/mok/host/mok_port_host.py:122,196).
What IS pinned by those files and implemented here: blocks of 32 along the contraction
dimension, E4M3 elements, one UE8M0 byte per block, and the ``[rows/128, cols/128, 32, 16]``
scale tensor with byte ``(r % 32) * 16 + (r / 32) * 4 + group`` inside a 128x128 block.

Scale rule fixed by this library (the published OCP-MX / "round the scale up" recipe):
    q     = amax / 448                      (IEEE fp32 division)
    e     = clamp(ceil(log2 q), -127, 127)  (exact, from q's bit pattern); amax == 0 -> -127
    byte  = e + 127
    elem  = RN-even, saturate-to-finite E4M3 of x * 2^-e
"""
from __future__ import annotations

import numpy as np

E4M3_MAX = 448.0


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bf16 (ties to even), returned as fp32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32).reshape(x.shape)
    return np.where(np.isnan(x), x, out)


def e8m0_from_amax(amax: np.ndarray) -> np.ndarray:
    amax = np.asarray(amax, dtype=np.float32)
    q = (amax / np.float32(448.0)).astype(np.float32)
    bits = q.view(np.uint32)
    exp = ((bits >> 23) & 0xFF).astype(np.int64)
    mant = (bits & 0x7FFFFF).astype(np.int64)
    normal = exp + (mant != 0)
    sub = (mant > 0x400000).astype(np.int64)
    e = np.where(exp == 0, sub, normal)
    return np.minimum(e, 254).astype(np.uint8)


def e8m0_inverse(byte: np.ndarray) -> np.ndarray:
    """2^(127 - byte) as fp32."""
    return np.ldexp(np.float32(1.0), 127 - byte.astype(np.int32)).astype(np.float32)


def e8m0_value(byte: np.ndarray) -> np.ndarray:
    """2^(byte - 127) as fp32."""
    return np.ldexp(np.float32(1.0), byte.astype(np.int32) - 127).astype(np.float32)


def float_to_e4m3(x: np.ndarray) -> np.ndarray:
    """cvt.rn.satfinite.e4m3.f32: nearest-even, |x| > 448 -> 448, NaN -> 0x7F."""
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float64)
    nan = np.isnan(a)
    a = np.where(nan, 0.0, a)
    a = np.minimum(a, 1e9)  # keep frexp finite; saturation handles the rest
    # exponent of the value, clamped to the subnormal exponent -6
    m, ex = np.frexp(a)           # a = m * 2^ex, m in [0.5, 1)
    e = np.maximum(ex - 1, -6)    # a in [2^e, 2^(e+1)) for normals
    quantum = np.ldexp(1.0, e - 3)
    steps = np.rint(a / quantum)  # ties to even; 0..16
    carry = steps >= 16
    e = np.where(carry, e + 1, e)
    steps = np.where(carry, 8, steps)
    is_sub = steps < 8            # only possible when e == -6
    code = np.where(is_sub, steps, ((e + 7).astype(np.int64) << 3) + (steps - 8)).astype(np.int64)
    code = np.where(code > 0x7E, 0x7E, code)
    code = np.where(a > 464.0, 0x7E, code)  # anything that would round past 448 saturates
    out = code.astype(np.uint8) | sign
    return np.where(nan, np.uint8(0x7F), out).astype(np.uint8)


def e4m3_to_float(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8)
    sign = np.where(b & 0x80, -1.0, 1.0)
    ex = ((b >> 3) & 0xF).astype(np.int32)
    man = (b & 7).astype(np.float64)
    normal = np.ldexp(1.0 + man / 8.0, ex - 7)
    sub = np.ldexp(man / 8.0, -6)
    v = np.where(ex == 0, sub, normal) * sign
    v = np.where((b & 0x7F) == 0x7F, np.nan, v)
    return v.astype(np.float32)


def scale_offsets(rows: int, cols: int) -> np.ndarray:
    """Byte offset of the scale of (row, 32-column group) in the [R/128, C/128, 32, 16] tensor."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    g = np.arange(cols // 32, dtype=np.int64)[None, :]
    return ((r >> 7) * (cols // 128) + (g >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (g & 3)


def pack_scales(sc_rg: np.ndarray) -> np.ndarray:
    """[rows, cols/32] scale bytes -> flat [rows/128, cols/128, 32, 16] tensor."""
    rows, groups = sc_rg.shape
    cols = groups * 32
    out = np.zeros(rows * groups, dtype=np.uint8)
    out[scale_offsets(rows, cols).reshape(-1)] = sc_rg.reshape(-1)
    return out.reshape(rows // 128, cols // 128, 32, 16)


def unpack_scales(sc: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """Inverse of pack_scales: -> [rows, cols/32]."""
    return np.asarray(sc, dtype=np.uint8).reshape(-1)[scale_offsets(rows, cols)]


def quantize(x: np.ndarray):
    """x fp32 (already bf16-representable) [rows, cols] -> (fp8 u8 [rows, cols], sc u8 packed)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    assert rows % 128 == 0 and cols % 128 == 0
    blocks = x.reshape(rows, cols // 32, 32)
    amax = np.fmax.reduce(np.abs(blocks), axis=2, initial=np.float32(0.0)).astype(np.float32)
    sc = e8m0_from_amax(amax)
    scaled = (blocks * e8m0_inverse(sc)[:, :, None]).astype(np.float32)
    q = float_to_e4m3(scaled).reshape(rows, cols)
    return q, pack_scales(sc)


def quantize_transposed(x: np.ndarray):
    """Blocks of 32 along the rows of x; outputs are laid out as the transpose [cols, rows]."""
    return quantize(np.ascontiguousarray(np.asarray(x, dtype=np.float32).T))


_E4M3_TABLE = None


def dequantize(q: np.ndarray, sc: np.ndarray) -> np.ndarray:
    """Element value (e4m3_to_float, through a 256-entry table of it) times the block's 2^(byte - 127)."""
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        _E4M3_TABLE = e4m3_to_float(np.arange(256, dtype=np.uint8))
    rows, cols = q.shape
    s = e8m0_value(unpack_scales(sc, rows, cols))
    vals = _E4M3_TABLE[np.asarray(q, dtype=np.uint8)]
    return (vals.reshape(rows, cols // 32, 32) * s[:, :, None]).reshape(rows, cols).astype(np.float32)
