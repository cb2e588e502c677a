"""Records what the REFERENCE's tensor contract loader (pipec/src/pipec2/tensor/contracts.py:
load_stage_tensor) answers for its own valid tensor section and for single mutations of it: the
failure paths under clause T-CONTRACT, and a few exact evaluations of placement / demand expressions.

Run in the build container, where the reference tree is mounted (it does not travel):

    python tests/golden/make_reference_tensor_cases.py <path to a checkout of the reference>

writes tests/golden/reference_tensor_cases.json. The valid section is the one the reference's tests
build (pipec/tests/pipec2/test_tensor_contracts.py:_valid_tensor); the mutations are listed below.
"""
import copy
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
if len(sys.argv) < 2:
    raise SystemExit("usage: " + Path(__file__).name + " <path to a checkout of the reference>")
REFERENCE = Path(sys.argv[1])
sys.path.insert(0, str(REFERENCE / "pipec" / "src"))
sys.path.insert(0, str(REFERENCE / "pipec" / "tests" / "pipec2"))

from pipec2.model import PipeLinkError  # noqa: E402
from pipec2.tensor import expr  # noqa: E402
from pipec2.tensor.contracts import load_stage_tensor  # noqa: E402
from test_tensor_contracts import _valid_tensor  # noqa: E402

# (name, path into the section, new value) or (name, path, "append", value) / (name, path, "dup")
MUTATIONS = [
    ("bad version", ["version"], "tensor-v1"),
    ("unknown import site", ["imports", 0, "sites"], "append", "missing_hook"),
    ("undeclared coordinate", ["exports", 0, "placements", 0, "components", "dp"], ["coord", "undeclared"]),
    ("undeclared binding", ["exports", 0, "placements", 0, "components", "dp"], ["bind", "partner_slot"]),
    ("binding used as coordinate", ["exports", 0, "placements", 0, "components", "dp"], ["coord", "slot"]),
    ("coordinate used as binding", ["exports", 0, "placements", 0, "components", "dp"], ["bind", "row"]),
    ("empty identity coordinate", ["exports", 0, "identity", "coords", 0, "hi"], 0),
    ("empty binding range", ["bindings", 1, "domain", "hi"], 0),
    ("empty demand coordinate", ["imports", 0, "demands", 0, "domain", 0, "hi"], 0),
    ("empty binding values", ["bindings", 0, "domain", "values"], []),
    ("binding domain name differs", ["bindings", 1, "domain", "name"], "different"),
    ("binding domain sort differs", ["bindings", 1, "domain", "sort"], "bits[4]"),
    ("relocatable lend without handle", ["imports", 0, "lends", 0, "location"], {"handle": None, "base": 0}),
    ("duplicate export", ["exports"], "dup"),
    ("duplicate import", ["imports"], "dup"),
    ("duplicate site", ["sites"], "dup"),
    ("duplicate binding", ["bindings"], "dup"),
    ("unknown operator", ["exports", 0, "placements", 0, "components", "dp"], ["frobnicate", ["coord", "row"]]),
    ("guard is not a predicate", ["exports", 0, "placements", 0, "guard"], ["coord", "row"]),
    ("unknown site guarantee", ["sites", 0, "guarantees"], ["converged", "sometimes"]),
    ("duplicate lend name", ["imports", 0, "lends", 1, "name"], "scratch"),
    ("rendezvous on a missing barrier", ["imports", 0, "rendezvous", 0, "barrier"], "nowhere"),
]


def mutated(case):
    obj = _valid_tensor()
    target = obj
    for part in case[1][:-1]:
        target = target[part]
    last = case[1][-1]
    if len(case) == 4 and case[2] == "append":
        target[last].append(case[3])
    elif case[2] == "dup":
        target[last].append(copy.deepcopy(target[last][0]))
    else:
        target[last] = copy.deepcopy(case[2])
    return obj


out = {"source": "pipec/src/pipec2/tensor/contracts.py:load_stage_tensor on pipec/tests/pipec2/test_tensor_contracts.py:_valid_tensor",
       "valid": _valid_tensor(), "cases": [], "evaluations": []}
stage = load_stage_tensor(_valid_tensor(), "$.tensor")
placement, demand = stage.exports[0].placements[0], stage.imports[0].demands[0]
valid = _valid_tensor()
for where, e, raw, env in (("exports[0].placements[0].components.dp", placement.components["dp"], valid["exports"][0]["placements"][0]["components"]["dp"], {"row": 127}),
                           ("exports[0].placements[0].components.column", placement.components["column"], valid["exports"][0]["placements"][0]["components"]["column"], {"tmem_base": 0, "col": 31, "slot": 1}),
                           ("exports[0].placements[0].components.column", placement.components["column"], valid["exports"][0]["placements"][0]["components"]["column"], {"tmem_base": 64, "col": 5, "slot": 0}),
                           ("exports[0].placements[0].guard", placement.guard, valid["exports"][0]["placements"][0]["guard"], {"row": 127}),
                           ("imports[0].demands[0].position", demand.position, valid["imports"][0]["demands"][0]["position"], {"c": 31})):
    out["evaluations"].append({"where": where, "expr": raw, "env": env, "value": expr.evaluate(e, env)})
for case in MUTATIONS:
    obj = mutated(case)
    try:
        load_stage_tensor(obj, "$.tensor")
        paths = []
    except PipeLinkError as err:
        assert all(f.clause_id == "T-CONTRACT" for f in err.failures)
        paths = [f.path for f in err.failures]
    out["cases"].append({"name": case[0], "path": case[1], "edit": list(case[2:]), "reference_paths": paths})
    print(case[0], "->", paths)
dst = ROOT / "tests" / "golden" / "reference_tensor_cases.json"
dst.write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
print(dst, dst.stat().st_size, "bytes")
