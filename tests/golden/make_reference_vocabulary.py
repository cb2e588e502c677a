"""Records what the reference's OWN annotation pass emits for the two vocabulary units under
tests/golden/sources/: small stage sources written here, in the reference's annotation spelling,
that between them use every form of the vocabulary its example stages use (endpoints with affine
and tensor-memory layouts, two-sided and one-shot barrier rings, named barriers, counters,
completion-only endpoints, exports and calls with wide signatures, claims in the positional, builder
and typed forms, register claims, variants with and without entries, topologies). The test packs
the same two sources with this repository's header and compares the declared sections.

Run in the build container, where the reference tree is mounted (it does not travel):

    python tests/golden/make_reference_vocabulary.py <path to a checkout of the reference>

writes tests/golden/reference_vocabulary_unit.json and tests/golden/reference_vocabulary_b_unit.json.
"""
import json
import os
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
if len(sys.argv) < 2:
    raise SystemExit("usage: " + Path(__file__).name + " <path to a checkout of the reference>")
REFERENCE = Path(sys.argv[1])
sys.path.insert(0, str(REFERENCE / "pipec" / "src"))
os.environ.setdefault("PIPEC_CUDA", "/usr/local/cuda")

from pipec2 import symbols  # noqa: E402  (the reference)
from pipec2.pack.assemble import assemble  # noqa: E402
from pipec2.pack.emit import compile_registry  # noqa: E402

PROFILE, TOOLKIT = "sm_100a", "cuda-13.3.0"


def emit(source: Path) -> dict:
    env = os.environ.copy()
    cuda = symbols.cuda_home(env)
    env["PATH"] = str(cuda / "bin") + os.pathsep + env.get("PATH", "")
    env["CUDA_VISIBLE_DEVICES"] = ""
    with tempfile.TemporaryDirectory() as tmp:
        comp = compile_registry(source, Path(tmp), includes=(), defines=(), nvcc_flags=(), profile=PROFILE,
                                toolkit=TOOLKIT, env=env)
        return assemble(comp.registry, profile=PROFILE, toolkit=TOOLKIT, provenance_inputs=comp.provenance_inputs,
                        math=comp.math)


for unit in ("vocabulary", "vocabulary_b"):
    manifest = emit(ROOT / "tests" / "golden" / "sources" / f"{unit}.cu")
    out = ROOT / "tests" / "golden" / f"reference_{unit}_unit.json"
    out.write_text(json.dumps(manifest, indent=1, sort_keys=True) + "\n")
    print(out, len(manifest["endpoints"]), "endpoints,", len(manifest["claims"]), "claims")
