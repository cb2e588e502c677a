"""Pipeline variants and single-mutation negatives of the three-stage GEMM, shared by the script
that records what the reference's linker front end answers (make_linker_golden.py) and by the test
that holds this repo's linker to those answers (tests/test_pipec2_cpu.py)."""
import copy

STAGES = ("load", "mma", "epilogue_bias_silu")

# name -> kwargs of pipelink_b200.stages.gemm3.build.pipeline_spec
SOLVE_CASES = {
    "default": {},
    "forced-depth-3": {"depth": 3},
    "seven-does-not-fit": {"values": (8, 7, 6, 5)},
    "small-values": {"values": (2, 3)},
}


def _endpoint(m, name):
    """Endpoints are selected by name: their order in a manifest is the packer's (by name), not the source's."""
    return next(e for e in m["endpoints"] if e["name"] == name)


def _set(stage, endpoint, path, value):
    def mutate(ms):
        node = _endpoint(ms[stage], endpoint)
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
    return mutate


# name -> mutation of [load, mma, epilogue] manifest dicts (deep copies)
NEGATIVE_CASES = {
    "missing-consumer": lambda ms: ms[1]["endpoints"].remove(_endpoint(ms[1], "operands")),
    "scope-differs": _set(1, "operands", ("scope",), "cluster"),
    "layout-stride-differs": _set(1, "operands", ("layout", "stride"), [[16384], [256], [1]]),
    "swizzle-differs": _set(1, "operands", ("layout", "swizzle"), {"B": 2, "M": 4, "S": 3}),
    "tmem-columns-differ": _set(2, "accumulator", ("layout", "cols"), 64),
    "tile-differs": _set(2, "accumulator", ("tile",), {"dtype": "f32", "shape": [128, 64]}),
    "empty-arrive-count-differs": _set(1, "operands", ("protocol", "empty", "arrive", "count"), 32),
    "ring-stride-differs": _set(1, "operands", ("ring", "stage_stride_bytes"), 16384),
}


def mutated(manifests: dict, name: str):
    ms = [copy.deepcopy(manifests[k]) for k in STAGES]
    NEGATIVE_CASES[name](ms)
    return ms
