"""The planning half of tensor imports, without a GPU: which route each cell of stages/tensor_import
gets and why the earlier ones were passed over, what the checker certifies and what it catches,
what a plan reserves, and the failures the reference names (docs/reference/tensor-imports.md
"Planning": routes tried in a fixed structural order, every proposal replayed against the terminal
demand, RESOURCE_ENVELOPE naming the missing facts, T-PLAN-RENDEZVOUS, T-PLAN-FRAME)."""
import copy
import json

import pytest

from pipelink_b200.pipec2 import link as linker, tensor, tensor_plan as tp
from pipelink_b200.pipec2.model import PipeLinkError
from pipelink_b200.stages.tensor_import import build as tb

ROUTES = {"tmem": "direct_receipt", "tmem_transposed": "staged_constructed", "smem": "shared_direct",
          "tmem_by_column": "staged_constructed", "smem_by_column": "shared_direct"}


def _members(cell, **changes):
    ms = [copy.deepcopy(tb.manifests()[u]) for u in tb.CELLS[cell]]
    return ms


def _pipe(cell):
    return tb.pipeline_spec(cell, [])["pipeline"]


def _plan(cell, edit=None):
    ms = _members(cell)
    if edit:
        edit(*ms)
    return tp.plan_pipeline(ms, _pipe(cell))


def _clauses(err):
    return [(f.clause_id, f.path) for f in err.value.failures]


@pytest.mark.parametrize("cell", sorted(ROUTES))
def test_every_cell_gets_its_route(cell):
    (rec,) = _plan(cell)
    assert rec["outcome"] == "MODEL_SAT" and rec["route"] == ROUTES[cell]
    tried = [(t["route"], t["outcome"]) for t in rec["tried"]]
    assert tried[-1] == (ROUTES[cell], "MODEL_SAT")
    assert [r for r, _ in tried] == list(tp.ROUTE_ORDER[:len(tried)])          # fixed structural order
    if ROUTES[cell] == "staged_constructed":
        assert tried[0] == ("direct_receipt", "BOUNDED_UNSAT")                 # the lanes hold other participants' elements
        assert rec["used"] == {"scratch_bytes": 65536, "barrier_generations": 3}
        assert {c["domain"]: c["extent"]["const"] for c in rec["claims"]} == {"smem": 65536, "named_barrier": 1}
        assert rec["unused_handles"] == []
    else:
        assert rec["used"] == {"scratch_bytes": 0, "barrier_generations": 2}
        assert [c["domain"] for c in rec["claims"]] == ["named_barrier"]      # an unused lend claims nothing
        assert rec["unused_handles"] == ["pipelink_ti_scratch"]


def test_staging_picks_the_conflict_free_shear():
    for cell in ("tmem_transposed", "tmem_by_column"):
        (rec,) = _plan(cell)
        load = rec["program"][-1]
        assert load["shear_modulus"] == 32 and load["bank_score"] == load["conflict_free_score"]
    # without a shear the transposed read walks one bank: 32-way conflicts on every load
    words = [[128 * p + t for t in range(32)] for p in range(4)]          # lane' = p, column' = t, no shear
    assert tp._bank_score(words) == 4
    words = [[128 * t + p for t in range(32)] for p in range(4)]          # lane' = t, column' = p, no shear
    assert tp._bank_score(words) == 4 * 32


@pytest.mark.parametrize("cell", ["tmem_transposed", "tmem_by_column"])
def test_staging_rounds_are_conflict_free_and_cover_the_scratch_exactly(cell):
    """The property the reference holds its staged routes to (pipec/tests/pipec2/test_tensor_construct.py:
    test_matrix_staging_is_conflict_free_without_changing_extent): per warp and per round every bank
    is hit once, and stores and loads visit exactly the words of the 64 KB scratch."""
    (rec,) = _plan(cell)
    store, load = rec["program"][1], rec["program"][3]
    visited = {}
    for step, var in ((store, "i"), (load, "p")):
        seen = set()
        for k in range(step["count"]):
            for warp in range(4):
                words = {tensor.evaluate(step["word"], {"t": 32 * warp + lane, var: k}) for lane in range(32)}
                assert len(words) == 32 and len({w % 32 for w in words}) == 32
                seen |= words
        visited[step["op"]] = seen
    assert visited["smem_store"] == visited["smem_load"] == set(range(65536 // 4))


def test_the_checker_replays_the_program_and_catches_a_wrong_one():
    ms = _members("tmem_transposed")
    pipe = _pipe("tmem_transposed")
    (rec,) = tp.plan_pipeline(ms, pipe)
    export = ms[0]["tensor"]["exports"][0]
    imp = ms[1]["tensor"]["imports"][0]
    site = dict(ms[1]["tensor"]["sites"][0], participants=128, warpgroup_aligned=True)
    conn = tp.Connection(export, imp, site)
    assert tp.certify(rec["program"], conn) == {"scratch_bytes": 65536, "barrier_generations": 1}
    # a load that forgets the shear reads another element
    bad = copy.deepcopy(rec["program"])
    bad[-1]["word"] = ["add", ["mulc", 128, ["coord", "p"]], ["coord", "t"]]
    with pytest.raises(tp.Infeasible) as err:
        tp.certify(bad, conn)
    assert err.value.outcome == "CHECK_FAILED" and "participant 0 position 1" in err.value.reason
    # reading scratch before the rendezvous that publishes it
    early = [s for s in rec["program"] if s["op"] != "rendezvous"]
    with pytest.raises(tp.Infeasible) as err:
        tp.certify(early, conn)
    assert "before the rendezvous" in err.value.reason
    # two participants storing to one word
    clash = copy.deepcopy(rec["program"])
    clash[1]["word"] = ["coord", "i"]
    with pytest.raises(tp.Infeasible) as err:
        tp.certify(clash, conn)
    assert "written twice" in err.value.reason


def test_c_lowering_is_held_to_the_exact_value():
    e = ["modc", ["sub", ["coord", "t"], ["const", 5]], 4]
    assert tensor.evaluate(e, {"t": 2}) == 1 and tp.c_value(e, {"t": 2}) == -3      # floor against truncation
    with pytest.raises(tp.Infeasible) as err:
        tp._value(e, {"t": 2})
    assert err.value.outcome == "LOWERING_UNSUPPORTED"
    assert tp._value(e, {"t": 9}) == 0
    text = tp.expr_to_c(["add", ["mulc", 128, ["coord", "t"]], ["toint", ["bxor", ["tobits", 7, ["coord", "p"]],
                                                                          ["tobits", 7, ["modc", ["coord", "t"], 32]]]]],
                        {"t": "pl_t", "p": "p"})
    assert text == "((128 * pl_t) + ((int)((((unsigned)(p)) ^ ((unsigned)((pl_t % 32)))))))"


def test_lends_too_small_name_what_is_missing():
    def small_scratch(_prod, cons):
        cons["tensor"]["imports"][0]["lends"][0]["extent"] = 32768
    with pytest.raises(PipeLinkError) as err:
        _plan("tmem_transposed", small_scratch)
    (f,) = err.value.failures
    assert (f.clause_id, f.path) == ("T-PLAN", "pipeline.tensor_connections.acc")
    assert f.detail["missing"] == {"smem_bytes": 65536}

    def two_generations(_prod, cons):
        cons["tensor"]["imports"][0]["lends"][1]["sync"]["generations"] = 2
    with pytest.raises(PipeLinkError) as err:
        _plan("tmem_by_column", two_generations)
    assert err.value.failures[0].detail["missing"] == {"barrier_generations": 3}
    # the same lend is enough where no staging is needed
    (rec,) = _plan("tmem", two_generations)
    assert rec["route"] == "direct_receipt"


def test_missing_outer_event_is_a_rendezvous_failure():
    def no_done(_prod, cons):
        cons["tensor"]["imports"][0]["rendezvous"].pop()
    with pytest.raises(PipeLinkError) as err:
        _plan("smem", no_done)
    assert _clauses(err) == [("T-PLAN-RENDEZVOUS", "tensor.imports.acc.rendezvous")]


def test_contract_and_model_failures():
    def other_dtype(_prod, cons):
        cons["tensor"]["imports"][0]["identity"] = dict(cons["tensor"]["imports"][0]["identity"], dtype="i32")
    with pytest.raises(PipeLinkError) as err:
        _plan("tmem", other_dtype)
    assert _clauses(err) == [("T-CONTRACT", "pipeline.tensor_connections.acc")]

    def half(prod, cons):
        for sec in (prod["tensor"]["exports"][0], cons["tensor"]["imports"][0]):
            sec["identity"] = dict(sec["identity"], dtype="bf16")
    with pytest.raises(PipeLinkError) as err:
        _plan("tmem", half)
    assert _clauses(err) == [("T-MODEL", "pipeline.tensor_connections.acc")]

    ms, pipe = _members("tmem"), _pipe("tmem")
    pipe["tensor_connections"].append(dict(pipe["tensor_connections"][0], name="again"))
    with pytest.raises(PipeLinkError) as err:
        tp.plan_pipeline(ms, pipe)
    assert _clauses(err) == [("T-CONTRACT", "pipeline.tensor_connections.again")]

    def overlapping(prod, _cons):
        prod["tensor"]["exports"][0]["placements"][0]["components"]["column"] = ["const", 0]
    with pytest.raises(PipeLinkError) as err:
        _plan("tmem", overlapping)
    assert _clauses(err)[0][0] in ("T-CONTRACT", "T-PLAN")


def test_tensor_memory_needs_a_warpgroup_aligned_role():
    def unaligned(prod, cons):
        for c in cons["claims"]:
            if c["domain"] == "warp":
                c["align"] = 1
        # a second role that owns warps: the importing role is no longer known to start at warp 0
        prod["stage"]["roles"]["feeder"] = {"entry": "feeder_role", "warps": 1}
    with pytest.raises(PipeLinkError) as err:
        _plan("tmem", unaligned)
    (f,) = err.value.failures
    assert f.clause_id == "T-PLAN" and f.detail["missing"] == {"role_warp_align": 4}
    (rec,) = _plan("smem", unaligned)            # shared memory has no such rule
    assert rec["route"] == "shared_direct"


def test_the_only_warp_owner_starts_at_warp_zero():
    """With one role in the whole pipeline its claim's alignment does not matter (the reference's
    one-epilogue cells: a four-warp epilogue whose warp claim has alignment 1)."""
    def unaligned(_prod, cons):
        for c in cons["claims"]:
            if c["domain"] == "warp":
                c["align"] = 1
    (rec,) = _plan("tmem", unaligned)
    assert rec["outcome"] == "MODEL_SAT"


def test_register_export_needs_a_frame():
    frame_export = {"name": "tile", "identity": tb.IDENTITY, "placements": [
        {"space": "regs", "components": {"participant": ["coord", "m"], "position": ["sub", ["const", 127], ["coord", "n"]]}}]}

    def regs(prod, cons, frame=True):
        prod["tensor"]["exports"] = [copy.deepcopy(frame_export)]
        if frame:
            cons["tensor"]["imports"][0]["lends"].append({"name": "acc_frame", "domain": "reg", "binding": "fixed", "extent": 128,
                                                          "purpose": "frame", "location": {"handle": "acc_frame"}})
    (rec,) = _plan("smem", regs)
    assert rec["route"] == "frame_local" and rec["program"][0]["op"] == "frame_load"
    text = tp.lower(rec, warp_lo=0, threads_in_role=128)
    assert "dest[p] = pl_frame[(127 - p)];" in text
    with pytest.raises(PipeLinkError) as err:
        _plan("smem", lambda p, c: regs(p, c, frame=False))
    assert _clauses(err) == [("T-PLAN-FRAME", "pipeline.tensor_connections.acc")]
    # a frame that lives in another participant needs a route this build does not have
    def crossed(prod, cons):
        regs(prod, cons)
        prod["tensor"]["exports"][0]["placements"][0]["components"] = {"participant": ["coord", "n"], "position": ["coord", "m"]}
    with pytest.raises(PipeLinkError) as err:
        _plan("smem", crossed)
    assert _clauses(err) == [("T-PLAN", "pipeline.tensor_connections.acc")]


@pytest.fixture(scope="module")
def linked(tmp_path_factory):
    out = tmp_path_factory.mktemp("ti")
    return out, tb.build(out, cells=("tmem", "tmem_transposed", "smem_by_column"))


def test_link_generates_certified_adapters_and_reserves_what_they_use(linked):
    out, results = linked
    direct, staged, shared = results["tmem"], results["tmem_transposed"], results["smem_by_column"]
    assert direct.dyn_smem_bytes == 16                       # the published TMEM base only: the scratch lend is unused
    assert direct.bindings["pipelink_ti_scratch"] == [0, "unused"]
    assert staged.dyn_smem_bytes == 65536 + 16 and shared.dyn_smem_bytes == 65536
    assert staged.bindings["pipelink_ti_barrier"][0] >= 1    # id 0 is the CTA-wide barrier
    for cell, r in results.items():
        text = (out / cell / "generated" / "tensor_adapters.cu").read_text()
        for fn in ("ti_import_acc", "ti_import_acc_ready", "ti_import_acc_done"):
            assert f'extern "C" __device__ void {fn}(' in text
        assert ("tcgen05.ld.sync.aligned.32x32b.x32.b32" in text) == cell.startswith("tmem")
        assert ("tcgen05.fence::before_thread_sync" in text) == cell.startswith("tmem")
        regs, stack, spill = r.observed
        assert 0 < regs <= 255 and spill == 0
        record = json.loads((out / cell / "link.json").read_text())["tensor"][0]
        assert record["route"] == ROUTES[cell] and record["plan_sha256"] == r.tensor[0]["plan_sha256"]
        assert (out / cell / "one_tu.cubin").stat().st_size > 0
    stub = (out / "tmem" / "generated" / "binding_stub.cu").read_text()
    assert "struct TiTileArgs;" in stub and "#include <pipelink/tensor_source.h>" in stub
    assert ("pipelink_call_tensor_produce(const struct TiTileArgs* a0, void* a1) { return ti_tmem_produce(a0, a1); }") in stub


def test_front_end_merges_the_reservations_into_the_solve():
    ms = _members("tmem_by_column")
    fe = linker.front_end(ms, _pipe("tmem_by_column"))
    assert fe["claims"]["pipelink_ti_scratch"]["rec"]["extent"]["const"] == 65536
    assert fe["claims"]["pipelink_ti_barrier"]["rec"]["domain"] == "named_barrier"
    assert all("pipelink_ti_scratch" != c["handle"] for c in ms[1]["claims"])      # the caller's manifests are left alone
    assert fe["tensor"][0]["route"] == "staged_constructed"
