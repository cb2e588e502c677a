"""Records the reference's 19 negative link fixtures as data: the base documents its test suite
builds (stage manifests + pipeline description, or symbol tables), each fixture's single mutation,
the clause and path the fixture expects, and what the REFERENCE's front end actually answers.

Run in the build container, where the reference tree is mounted (it does not travel):

    python tests/golden/make_reference_negatives.py <path to a checkout of the reference>

writes tests/golden/reference_negative_fixtures.json. The fixtures live in
pipec/tests/pipec2/fixtures/negative/*.json; the bases come from the builders in
pipec/tests/pipec2/test_negative_fixtures.py (BASES), run here unmodified.
"""
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
if len(sys.argv) < 2:
    raise SystemExit("usage: " + Path(__file__).name + " <path to a checkout of the reference>")
REFERENCE = Path(sys.argv[1])
sys.path.insert(0, str(REFERENCE / "pipec" / "src"))
sys.path.insert(0, str(REFERENCE / "pipec" / "tests" / "pipec2"))

import test_negative_fixtures as ref  # noqa: E402  (the reference's own test module)

out = {"source": "pipec/tests/pipec2/fixtures/negative + test_negative_fixtures.py:BASES", "bases": {}, "cases": []}
for name, make in ref.BASES.items():
    out["bases"][name] = make()
for path in sorted(ref.FIXTURE_DIR.glob("*.json")):
    case, raw = ref._load_case(path.name)
    failures = ref._run_case(case, raw)
    mutation = case["mutation"]
    out["cases"].append({
        "file": path.name, "name": case["name"], "base": case["base"], "phase": case["phase"],
        "channel": case.get("channel"), "stage_index": case.get("stage_index", 0),
        "paths": mutation["paths"] if "paths" in mutation else [mutation["path"]], "value": mutation["value"],
        "expected_clause": case["expected_clause"], "expected_path": case["expected_path"],
        "reference_failures": [[f.clause_id, f.path, f.message] for f in failures]})
dst = ROOT / "tests" / "golden" / "reference_negative_fixtures.json"
dst.write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
print(dst, len(out["cases"]), "cases,", dst.stat().st_size, "bytes")
