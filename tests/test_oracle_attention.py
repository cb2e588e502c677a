"""The attention oracle's fixture generator against vectors recorded from the reference's own
stream definition (tests/golden/philox_f2_streams.json, made by tests/golden/make_stream_golden.py),
plus self-consistency of its row evaluation."""
import json
from pathlib import Path

import numpy as np

from oracle import attention as oa

GOLDEN = json.loads((Path(__file__).parent / "golden" / "philox_f2_streams.json").read_text())


def _bits(values_f32):
    return (np.asarray(values_f32, np.float32).view(np.uint32) >> 16).astype(np.int64)


def test_stream_key_matches_the_reference_namespace():
    assert oa.SEED == GOLDEN["seed"] and oa.NAMESPACE_ATTENTION == GOLDEN["namespace_id"]


def test_philox_words_and_bf16_elements_match_recorded_reference_values():
    for numeric_case, role, j, word, bits in GOLDEN["records"]:
        block, lane = divmod(j, 4)
        w = oa.philox4x32_10((np.uint64(block & 0xFFFFFFFF), np.uint64(block >> 32), np.uint64(numeric_case), np.uint64(role)),
                             (oa.SEED, oa.NAMESPACE_ATTENTION))
        assert int(w[lane]) == word, (numeric_case, role, j)
        if j < (1 << 22):
            got = oa.philox_bf16(j + 1, numeric_case, role)[j]
            assert int(_bits([got])[0]) == bits, (numeric_case, role, j)


def test_a_run_of_4096_elements_matches_bit_for_bit():
    run = GOLDEN["run"]
    got = _bits(oa.philox_bf16(len(run["bf16_bits"]), run["numeric_case"], run["role"]))
    assert np.array_equal(got, np.asarray(run["bf16_bits"], np.int64))


def test_reference_rows_agree_with_a_dense_softmax():
    rng = np.random.default_rng(0)
    S, Hq, Hkv, D = 64, 4, 2, 128
    q, k, v = (rng.standard_normal((S, h, D)).astype(np.float32) for h in (Hq, Hkv, Hkv))
    rows = [0, 1, 31, 63]
    out, lse = oa.reference_rows(q, k, v, rows, 0.1)
    for i, r in enumerate(rows):
        for h in range(Hq):
            s = (k[: r + 1, h // 2].astype(np.float64) @ q[r, h].astype(np.float64)) * 0.1
            p = np.exp(s - s.max())
            assert np.allclose(out[i, h], (p @ v[: r + 1, h // 2].astype(np.float64)) / p.sum(), atol=1e-9)
            assert abs(lse[h, i] - (s.max() + np.log(p.sum()))) < 1e-9
