"""Records words and bf16 elements of the reference's Philox fixture streams for the attention
family (namespace F2; roles 1 = Q, 2 = K, 3 = V), as its own Python restatement produces them.

Run in the build container, where the reference tree is mounted (it does not travel):

    python tests/golden/make_stream_golden.py <path to a checkout of the reference>

writes tests/golden/philox_f2_streams.json. The bf16 element is the reference's single rounding
of the binary64 value -2 + 4u (evaluator/harness/parity/streams.py `_bfloat16_bits_rne`, the same
rule as `fill_philox_bf16`, campaigns/attention/src/slot/fixtures.cuh:96-102).
"""
import json
import sys
from pathlib import Path

if len(sys.argv) < 2:
    raise SystemExit("usage: " + Path(__file__).name + " <path to a checkout of the reference>")
REFERENCE = Path(sys.argv[1])
sys.path.insert(0, str(REFERENCE))

from evaluator.harness.parity import streams  # noqa: E402  (the reference)

cases = [(0, 1), (0, 2), (0, 3), (7, 1), (17, 3)]
indices = list(range(0, 48)) + [255, 256, 1023, 4099, 65537, (1 << 20) + 3, (1 << 32) + 5, (1 << 34) + 2]
records = []
for numeric_case, role in cases:
    for j in indices:
        word = streams.word_at("F2", numeric_case, role, j)
        value = -2.0 + 4.0 * streams.uniform01(word)
        records.append([numeric_case, role, j, word, streams._bfloat16_bits_rne(value)])
# a longer run, to catch any element whose float32 detour would round differently from binary64
run = [streams._bfloat16_bits_rne(-2.0 + 4.0 * streams.uniform01(streams.word_at("F2", 3, 2, j))) for j in range(4096)]
out = {"namespace": "F2", "namespace_id": streams.NAMESPACE_IDS["F2"], "seed": streams.PHILOX_SEED,
       "records": records, "run": {"numeric_case": 3, "role": 2, "bf16_bits": run}}
target = Path(__file__).with_name("philox_f2_streams.json")
target.write_text(json.dumps(out, separators=(",", ":")) + "\n")
print(target, len(records), "records")
