"""The manifest's tensor section against the reference's loader: its own valid section passes, single
mutations of it fail at the paths the reference reports (tests/golden/make_reference_tensor_cases.py
recorded them), placement and demand expressions evaluate to the reference's values, and an import
is checked against the export it names."""
import copy
import json
from pathlib import Path

import pytest

from pipelink_b200.pipec2 import tensor

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_tensor_cases.json").read_text())


def _apply(case):
    obj = copy.deepcopy(GOLDEN["valid"])
    target = obj
    for part in case["path"][:-1]:
        target = target[part]
    last, edit = case["path"][-1], case["edit"]
    if len(edit) == 2 and edit[0] == "append":
        target[last].append(edit[1])
    elif edit == ["dup"]:
        target[last].append(copy.deepcopy(target[last][0]))
    else:
        target[last] = copy.deepcopy(edit[0])
    return obj


def test_the_reference_section_is_well_formed():
    assert tensor.validate_section(copy.deepcopy(GOLDEN["valid"]), "2.2") == []
    assert [f[1] for f in tensor.validate_section(GOLDEN["valid"], "2.0-draft")] == ["$.tensor"]


@pytest.mark.parametrize("case", GOLDEN["cases"], ids=[c["name"] for c in GOLDEN["cases"]])
def test_mutations_fail_where_the_reference_says(case):
    got = tensor.validate_section(_apply(case), "2.2")
    assert got and all(f[0] == "T-CONTRACT" for f in got)
    assert sorted({f[1] for f in got}) == sorted(set(case["reference_paths"]))


def test_expressions_evaluate_as_the_reference_does():
    for ev in GOLDEN["evaluations"]:
        assert tensor.evaluate(ev["expr"], ev["env"]) == ev["value"], ev
    coords, binds = {"row": "int", "col": "int"}, {"tmem_base": "int", "slot": "int"}
    column = GOLDEN["valid"]["exports"][0]["placements"][0]["components"]["column"]
    assert tensor.sort_of(column, coords, binds) == "int"
    assert tensor.sort_of(["lt", column, ["const", 512]], coords, binds) == "pred"
    # every (slot, col) of both admitted bases lands on its own column: the placement is injective
    cols = {tensor.evaluate(column, {"tmem_base": 0, "slot": s, "col": c}) for s in range(2) for c in range(32)}
    assert cols == set(range(64))
    assert tensor.evaluate(["shlc", ["tobits", 8, ["const", 200]], 1], {}) == (200 << 1) & 255
    assert tensor.evaluate(["select", ["le", ["const", 3], ["const", 3]], ["const", 7], ["const", 9]], {}) == 7
    with pytest.raises(tensor.ExprError):
        tensor.sort_of(["add", ["lt", ["const", 1], ["const", 2]], ["const", 1]], {}, {})
    with pytest.raises(tensor.ExprError):
        tensor.evaluate(["tobits", 4, ["const", 16]], {})


def test_an_import_is_checked_against_its_export():
    export, imp = GOLDEN["valid"]["exports"][0], GOLDEN["valid"]["imports"][0]
    assert tensor.check_import(export, imp) == []
    other = copy.deepcopy(imp)
    other["identity"]["dtype"] = "bf16"
    assert [f[1] for f in tensor.check_import(export, other)] == ["identity.dtype"]
    narrower = copy.deepcopy(imp)
    narrower["identity"]["coords"][1]["hi"] = 16
    assert [f[1] for f in tensor.check_import(export, narrower)] == ["identity.coords"]
    partial = copy.deepcopy(imp)
    del partial["demands"][0]["identity_coords"]["col"]
    assert [f[1] for f in tensor.check_import(export, partial)] == ["demands[0].identity_coords"]
