"""Records what the reference's OWN annotation pass emits for the stage sources of its
`examples/one-epilogue-many-producers` that make up the two sm_100a cells of its build.py: the epilogue that
imports an accumulator tile and a row-scale vector (consumer/epilogue.cu), the provider that exports the row
scales from shared memory (providers/rowscale/rowscale.cu) and the accumulator provider
(providers/accumulator/producer_source.cu) packed twice, exporting the tile from tensor memory
(-DPL_EXPORT_TMEM) and from swizzled shared memory (-DPL_EXPORT_SMEM); its mainloop includes CUTLASS, which the
example takes from a submodule that is not checked out: pass any recent CUTLASS include tree. A smaller
tensor-memory provider (producer_m128.cu) is recorded as well. These are the units that use the tensor
annotations (PL_SITE, PL_IMPORT_TENSOR, PL_EXPORT_TENSOR, PL_BINDING): maps written as C++ lambdas, tabulated
by the pass and fitted to expressions.

Run in the build container, where the reference tree is mounted (it does not travel):

    python tests/golden/make_reference_one_epilogue.py <path to a checkout of the reference> <CUTLASS include dir>

writes tests/golden/reference_one_epilogue_units.json.
"""
import json
import os
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
if len(sys.argv) < 3:
    raise SystemExit("usage: " + Path(__file__).name + " <path to a checkout of the reference> <CUTLASS include dir>")
REFERENCE, CUTLASS = Path(sys.argv[1]), Path(sys.argv[2])
sys.path.insert(0, str(REFERENCE / "pipec" / "src"))
os.environ.setdefault("PIPEC_CUDA", "/usr/local/cuda")

from pipec2 import symbols  # noqa: E402  (the reference)
from pipec2.pack.assemble import assemble  # noqa: E402
from pipec2.pack.emit import compile_registry  # noqa: E402

PROFILE, TOOLKIT = "sm_100a", "cuda-13.3.0"
EXAMPLE = REFERENCE / "examples" / "one-epilogue-many-producers"
TCGEN05 = {"PL_TILE_N": "128", "PL_MMA_M": "128"}          # the defines of the example's params.py for this profile
UNITS = {"consumer": ("consumer/epilogue.cu", {}), "rowscale": ("providers/rowscale/rowscale.cu", {}),
         "producer_m128": ("providers/accumulator/producer_m128.cu", {}),
         "acc_tmem": ("providers/accumulator/producer_source.cu", {**TCGEN05, "PL_EXPORT_TMEM": "1"}),
         "acc_smem": ("providers/accumulator/producer_source.cu", {**TCGEN05, "PL_EXPORT_SMEM": "1"})}


def emit(source: Path, defines: dict) -> dict:
    env = os.environ.copy()
    cuda = symbols.cuda_home(env)
    env["PATH"] = str(cuda / "bin") + os.pathsep + env.get("PATH", "")
    env["CUDA_VISIBLE_DEVICES"] = ""
    with tempfile.TemporaryDirectory() as tmp:
        comp = compile_registry(source, Path(tmp), includes=(CUTLASS,), defines=tuple(f"{k}={v}" for k, v in defines.items()), nvcc_flags=(), profile=PROFILE,
                                toolkit=TOOLKIT, env=env)
        return assemble(comp.registry, profile=PROFILE, toolkit=TOOLKIT, provenance_inputs=comp.provenance_inputs,
                        math=comp.math)


record = {"units": {name: {"source": "examples/one-epilogue-many-producers/" + rel, "defines": defines,
                           "manifest": emit(EXAMPLE / rel, defines)}
                    for name, (rel, defines) in UNITS.items()}}
out = ROOT / "tests" / "golden" / "reference_one_epilogue_units.json"
out.write_text(json.dumps(record, indent=None, sort_keys=True) + "\n")
print(out, out.stat().st_size, "bytes")
