"""Call channels end to end without a GPU: a role-less provider and a four-warp caller packed
separately (stages/hello), the trampoline the link generates from the two declarations, the device
link, and what the link refuses (the reference's first tutorial builds the same pair:
examples/hello-callable, docs/reference/annotations.md:58-90)."""
import copy

import pytest

from pipelink_b200.pipec2 import link as linker
from pipelink_b200.pipec2.model import PipeLinkError
from pipelink_b200.stages.hello import build as hb


def _front_end(provider, caller):
    stages = [m for m in (provider, caller) if m is not None]
    return linker.front_end(stages, hb.pipeline_spec([])["pipeline"])


def _clauses(err):
    return [(f.clause_id, f.path) for f in err.value.failures]


def test_annotations_state_both_ends_of_the_call():
    ms = hb.manifests()
    provider, caller = ms["provider"], ms["caller"]
    assert provider["stage"]["roles"] == {} and provider["params"]["bytes"] == 0
    assert provider["stage"]["exports"]["scale"]["symbol"] == "hello_scale"
    (pe,), (ce,) = provider["endpoints"], caller["endpoints"]
    assert pe["owner_role"] is None and pe["direction"] == "consume"      # a callee never names its caller's role
    assert ce["owner_role"] == "call" and ce["direction"] == "produce"
    import hashlib
    for ep, symbol in ((pe, "hello_scale"), (ce, "pipelink_call_scale")):
        decl = f'extern "C" __device__ float {symbol}(float);'       # the declaration, spelled from the function's type
        assert ep["protocol"] == {"kind": "call", "export": "scale", "signature": "float(float)", "decl": decl,
                                  "decl_sha256": hashlib.sha256(decl.encode()).hexdigest()}
    assert provider["stage"]["exports"]["scale"]["decl"] == pe["protocol"]["decl"]
    assert [c["handle"] for c in caller["claims"]] == ["pipelink_call_warps"]      # the role's own warp claim, derived
    assert caller["stage"]["roles"]["call"]["warps"] == 4
    assert caller["params"]["bytes"] == 24 and [m["name"] for m in caller["params"]["members"]] == ["input", "output", "count"]


def test_front_end_pairs_the_call_and_plans_the_trampoline():
    ms = hb.manifests()
    fe = _front_end(ms["provider"], ms["caller"])
    (e,) = fe["expansions"]
    assert e["kind"] == "call" and (e["producer"], e["consumer"]) == ("hello.caller", "hello.provider")
    assert e["trampoline"] == {"caller": "pipelink_call_scale", "provider": "hello_scale", "signature": "float(float)"}


def test_link_generates_the_trampoline_and_an_image(tmp_path):
    r = hb.build(tmp_path)
    stub = (tmp_path / "link" / "generated" / "binding_stub.cu").read_text()
    assert 'extern "C" __device__ float hello_scale(float);' in stub
    assert 'extern "C" __device__ float pipelink_call_scale(float a0) { return hello_scale(a0); }' in stub
    dispatch = (tmp_path / "link" / "generated" / "dispatch.cu").read_text()
    assert "if (warp >= 0 && warp < 4) hello_call(p.bytes + 0, 0u);" in dispatch
    assert r.threads == 128 and r.dyn_smem_bytes == 0
    regs, stack, spill = r.observed
    assert 0 < regs <= 64 and stack == 0 and spill == 0          # the call was inlined: no frame
    assert (tmp_path / "link" / "pipeline.cubin").stat().st_size > 0 and (tmp_path / "link" / "one_tu.cubin").stat().st_size > 0


def test_the_package_records_the_trampoline_as_an_undefined_symbol(tmp_path):
    from pipelink_b200.pipec2 import container, pack
    pack.pack_cu(hb.HERE / "caller.cu", None, tmp_path / "caller.plink")
    m, _ = container.read(tmp_path / "caller.plink")
    assert "pipelink_call_scale" in m["symbols"]["undefined"]
    # without the provider nothing defines it: the channel has one end
    with pytest.raises(PipeLinkError) as err:
        _front_end(None, m)
    assert _clauses(err) == [("L-PAIR", "channels.scale")]


@pytest.mark.parametrize("field,value", [("signature", "float(float, int)"), ("export", "other")])
def test_ends_that_disagree_do_not_link(field, value):
    ms = hb.manifests()
    caller = copy.deepcopy(ms["caller"])
    caller["endpoints"][0]["protocol"][field] = value
    with pytest.raises(PipeLinkError) as err:
        _front_end(ms["provider"], caller)
    assert _clauses(err) == [("L-PROTO", "channels.scale.protocol")]


def test_a_provider_without_the_export_does_not_link():
    ms = hb.manifests()
    provider = copy.deepcopy(ms["provider"])
    provider["stage"]["exports"] = {}
    with pytest.raises(PipeLinkError) as err:
        _front_end(provider, ms["caller"])
    assert _clauses(err) == [("L-SYM", "channels.scale.protocol.export")]


def test_signatures_are_spelled_from_the_declarations(tmp_path):
    """The closed set of types a call may carry: scalars, pointers to them, const; integers are spelled
    by their fixed-width names, as the reference's pass spells them."""
    src = tmp_path / "sig.cu"
    src.write_text('#include <pipelink/stage.hpp>\n'
                   'extern "C" __device__ void f(const float* a, unsigned long long* b, int n, double s);\n'
                   'extern "C" __device__ void role(const void* params, unsigned variant);\n'
                   'PL_STAGE("t.sig", "1.0.0");\nPL_NO_PARAMS();\nPL_ROLE(r, role, 1);\n'
                   'PL_CALL(ch, f, pl::produce, "r", "impl");\n')
    from pipelink_b200.pipec2 import codegen, pack
    m = pack.emit_manifest(src)
    proto = m["endpoints"][0]["protocol"]
    assert proto["signature"] == "void(const float*, uint64_t*, int32_t, double)" and proto["export"] == "impl"
    text = codegen.binding_stub({}, [{"caller": "f", "provider": "g", "signature": proto["signature"]}])
    assert ('extern "C" __device__ void f(const float* a0, uint64_t* a1, int32_t a2, double a3) { g(a0, a1, a2, a3); }'
            in text)
