"""The reference's example SOURCES through this repo's annotation header: `<pipelink/stage.hpp>` here
accepts the reference's spelling of the declarations (pl::endpoint("name", direction, "role"),
pl::affine, pl::mbarrier{pl::side{...}, ...}, pl::claim(...).extent(...), pl::topology{...}, PL_CALL),
so a stage written for the reference packs here unchanged. Each unit's manifest must equal, section by
section, the one the reference's own annotation pass emitted for the same file (recorded in
tests/golden/reference_*.json by running the reference). The sources live in the reference tree, which
exists in the build container only: without it these tests are skipped (PIPELINK_REFERENCE overrides
the path)."""
import json
import os
from pathlib import Path

import pytest

from pipelink_b200.pipec2 import pack
from pipelink_b200.pipec2.model import PipeLinkError

REFERENCE = Path(os.environ.get("PIPELINK_REFERENCE", "/root/reference"))
GOLDEN = Path(__file__).parent / "golden"
pytestmark = pytest.mark.skipif(not (REFERENCE / "examples" / "ring-pipeline" / "src" / "producer.cu").exists(),
                                reason="the reference's sources are not on this machine")
SECTIONS = ("stage", "endpoints", "claims", "topology")


def _same(mine, theirs):
    for section in SECTIONS:
        assert mine[section] == theirs[section], section
    for key in ("type", "bytes", "align"):
        assert mine["params"][key] == theirs["params"][key], f"params.{key}"


@pytest.mark.parametrize("index,name", [(0, "producer"), (1, "consumer")])
def test_ring_pipeline_sources_emit_the_reference_manifests(index, name):
    golden = json.loads((GOLDEN / "reference_ring_pipeline.json").read_text())
    _same(pack.emit_manifest(REFERENCE / "examples" / "ring-pipeline" / "src" / f"{name}.cu"), golden["manifests"][index])


@pytest.mark.parametrize("index,name", [(0, "provider"), (1, "caller")])
def test_hello_callable_sources_emit_the_reference_manifests(index, name):
    golden = json.loads((GOLDEN / "reference_hello_callable.json").read_text())
    _same(pack.emit_manifest(REFERENCE / "examples" / "hello-callable" / "src" / f"{name}.cu"), golden["manifests"][index])


GALLERY = json.loads((GOLDEN / "reference_contract_gallery.json").read_text())


@pytest.mark.parametrize("name", sorted(GALLERY["cases"]))
def test_contract_gallery_sources_pack_as_the_reference_packs_them(name):
    case = GALLERY["cases"][name]
    source = REFERENCE / case["source"]
    if case["phase"] == "pack":       # refused while packing: the same clause at the same path
        with pytest.raises(PipeLinkError) as err:
            pack.emit_manifest(source)
        assert [(f.clause_id, f.path) for f in err.value.failures] == [(f["clause"], f["path"]) for f in case["reference"]]
        return
    _same(pack.emit_manifest(source), case["manifest"])


def test_ring_pipeline_sources_pack_and_link_into_an_image(tmp_path):
    """Pack the reference's two ring-pipeline sources with this toolchain (annotations, LTO payload,
    undefined-symbol scan), link them with the pipeline description of its build.py and device-link the
    image: the whole path of `pipec2 pack` + `pipec2 link` on sources written for the reference. The image
    is not launched here (the sources are not this repo's to ship)."""
    from pipelink_b200.pipec2 import link as linker
    golden = json.loads((GOLDEN / "reference_ring_pipeline.json").read_text())
    src = REFERENCE / "examples" / "ring-pipeline" / "src"
    for name in ("producer", "consumer"):
        pack.pack_cu(src / f"{name}.cu", None, tmp_path / f"{name}.plink")
    doc = json.loads(json.dumps(golden["pipelines"]["solved"]))
    doc["pipelink_abi"]["target"]["toolkit"] = "cuda-12.9"
    for st, name in zip(doc["pipeline"]["stages"], ("producer", "consumer")):
        st["artifact_path"] = f"{name}.plink"
    (tmp_path / "pipeline.json").write_text(json.dumps(doc))
    r = linker.link(tmp_path / "pipeline.json", tmp_path / "link")
    want = golden["reference"]["solved"]
    assert (r.threads, r.dyn_smem_bytes) == (want["threads"], want["dyn_smem_bytes"])
    assert r.bindings["pipelink_ring_depth"][0] == want["depths"]["pipelink_ring_depth"]
    regs, stack, spill = r.observed
    assert 0 < regs <= 255 and spill == 0
    assert (tmp_path / "link" / "pipeline.cubin").stat().st_size > 0
    dispatch = (tmp_path / "link" / "generated" / "dispatch.cu").read_text()
    assert "ring_producer(p.bytes" in dispatch and "ring_consumer(p.bytes" in dispatch


HOPPER = json.loads((GOLDEN / "reference_hopper_gemm_split.json").read_text())


def _cutlass_include():
    """Any recent CUTLASS include tree (the example's own is a submodule that is not checked out): only
    declarations are needed for the manifest pass."""
    for module in ("flashinfer", "tilelang"):
        import importlib.util
        spec = importlib.util.find_spec(module)      # located, not imported
        if spec is None or not spec.origin:
            continue
        root = Path(spec.origin).parent
        for sub in ("data/cutlass/include", "3rdparty/cutlass/include"):
            if (root / sub / "cutlass" / "arch" / "barrier.h").exists():
                return root / sub
    return None


@pytest.mark.parametrize("name", sorted(HOPPER["manifests"]))
def test_hopper_gemm_split_sources_emit_the_reference_manifests(name):
    """Hopper units: only their host projection is compiled (as CUDA for sm_90a where a unit insists on it)."""
    cutlass = _cutlass_include()
    if cutlass is None:
        pytest.skip("no CUTLASS include tree on this machine")
    example = REFERENCE / "examples" / "hopper-gemm-split"
    _same(pack.emit_manifest(example / "src" / f"{name}.cu", includes=(str(cutlass), str(example / "src")), profile="sm_90a"),
          HOPPER["manifests"][name])


PROFILE_CONSUMER = json.loads((GOLDEN / "reference_profile_consumer.json").read_text())


@pytest.mark.parametrize("index,name", [(1, "instruction1"), (2, "instruction2")])
def test_profile_consumer_instruction_sources_emit_the_reference_manifests(index, name):
    """Named-barrier and counter endpoints, nested layout trees, positional PL_CLAIM with a phase lifetime,
    PL_DESCRIPTOR, a dynamic cluster, a namespace-qualified params type. (The third unit of the example, its
    scheduler, declares a host owner with PL_HOST_* annotations this header does not have.)"""
    example = REFERENCE / "examples" / "profile-consumer" / "src"
    _same(pack.emit_manifest(example / f"{name}.cu", includes=(str(example), str(REFERENCE / "pipec/src/pipec2/host/include"))),
          PROFILE_CONSUMER["manifests"][index])


ONE_EPILOGUE = json.loads((GOLDEN / "reference_one_epilogue_units.json").read_text())["units"]


def _one_epilogue_unit(name, cutlass):
    unit = ONE_EPILOGUE[name]
    mine = pack.emit_manifest(REFERENCE / unit["source"], includes=(str(cutlass),),
                              defines=[f"{k}={v}" for k, v in unit["defines"].items()], profile=unit["profile"])
    _same(mine, unit["manifest"])
    assert mine["tensor"] == unit["manifest"]["tensor"], name


def test_one_epilogue_sources_emit_the_reference_tensor_sections():
    """The tensor annotations (PL_SITE, PL_IMPORT_TENSOR, PL_EXPORT_TENSOR, PL_BINDING, PL_TYPE with members):
    the maps are C++ lambdas; this header finds their forms itself and must print the expressions the reference's
    pass fitted: affine ones (the tensor-memory placement comes out of a CUTLASS tiled-MMA layout, offset by a
    bound base column), an XOR-linear one (the 128-byte-swizzled shared-memory tile of the second cell) and a bit
    permutation printed as integer fields (the Hopper provider's warpgroup-MMA register fragment).
    The units compile side by side: the providers' mainloops take most of a minute each."""
    from concurrent.futures import ThreadPoolExecutor
    cutlass = _cutlass_include()
    if cutlass is None:
        pytest.skip("no CUTLASS include tree on this machine")
    with ThreadPoolExecutor(len(ONE_EPILOGUE)) as pool:
        for job in [pool.submit(_one_epilogue_unit, name, cutlass) for name in sorted(ONE_EPILOGUE)]:
            job.result()
