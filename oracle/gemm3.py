"""CPU oracle for the three-stage MXFP8 GEMM (BASELINE config 0) — TEST INFRASTRUCTURE.

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import
this module.

Same role as the reference's examples/hopper-gemm-split/oracle.py:112-127 (seeded operands, a
library GEMM as the expected result, ``compare`` with rtol/atol) with the configuration BASELINE
names: A, B ~ N(0,1) (seed 0) quantised to E4M3 with one UE8M0 scale per 32 elements along K,
bias ~ N(0, 0.1), out = bf16(silu(A_q . B_q^T + bias)). Tolerance: the evaluator's GEMM gate
rtol 1e-2, atol 1e-3 (evaluator/harness/parity/constants.py:49-52) on top of bf16 output rounding.
"""
from __future__ import annotations

import numpy as np
import torch

from . import mxfp8


def make_case(M=1024, N=1024, K=1024, seed=0):
    g = torch.Generator().manual_seed(seed)
    a = mxfp8.bf16_round(torch.randn(M, K, generator=g).numpy())
    b = mxfp8.bf16_round(torch.randn(N, K, generator=g).numpy())
    bias = mxfp8.bf16_round((torch.randn(N, generator=g) * 0.1).numpy())
    aq, asc = mxfp8.quantize(a)
    bq, bsc = mxfp8.quantize(b)
    return dict(a=a, b=b, bias=bias, aq=aq, asc=asc, bq=bq, bsc=bsc)


def expected(case):
    ad = torch.from_numpy(mxfp8.dequantize(case["aq"], case["asc"]))
    bd = torch.from_numpy(mxfp8.dequantize(case["bq"], case["bsc"]))
    acc = torch.matmul(ad.double(), bd.double().T) + torch.from_numpy(case["bias"]).double()[None, :]
    out = acc / (1.0 + torch.exp(-acc))
    return mxfp8.bf16_round(out.float().numpy())


def compare(ref, got, rtol=1e-2, atol=1e-3):
    """allclose with a bf16 ulp of slack (both sides are bf16-rounded)."""
    ref, got = np.asarray(ref, np.float64), np.asarray(got, np.float64)
    err = np.abs(ref - got)
    tol = atol + rtol * np.abs(ref) + np.abs(ref) * 2.0 ** -7
    rel_l2 = float(np.sqrt((err ** 2).sum() / (ref ** 2).sum()))
    return dict(violations=int((err > tol).sum()), max_abs=float(err.max()), rel_l2=rel_l2)
