"""``pipec2 pack``: stage source + manifest -> ``.plink``.

The reference emits the manifest by running the translation unit's host projection of its
``PL_*`` annotations (docs/reference/pack-and-link.md:23-43). This build keeps the manifest as a
JSON document beside the source (``<stage>.manifest.json``, same schema 3.0 records the
annotations would register) and does the two remaining pack steps: compile the LTO payload
(``nvcc -dc -gencode arch=compute_100a,code=lto_100a``) and assemble the canonical container.
"""
from __future__ import annotations

import hashlib
import json
import tempfile
from pathlib import Path

from . import container, jitlink, schema
from .profile import PROFILES


def pack_cu(source, manifest_path=None, out=None, profile="sm_100a", includes=(), defines=()):
    source = Path(source)
    manifest_path = Path(manifest_path) if manifest_path else source.with_suffix(".manifest.json")
    manifest = json.loads(manifest_path.read_text())
    manifest["pipelink_abi"]["target"]["profile"] = profile
    manifest["pipelink_abi"]["target"]["lto_arch"] = PROFILES[profile]["lto_arch"]
    schema.validate_manifest(manifest, where=manifest["stage"].get("id", str(source)))
    with tempfile.TemporaryDirectory() as tmp:
        obj = Path(tmp) / "stage.o"
        jitlink.compile_lto(str(source), str(obj), PROFILES[profile], includes, defines)
        payload = obj.read_bytes()
    # provenance as the reference records it (pipec/src/pipec2/schema.py:1015-1030): how the
    # manifest came to be and the digests of what it was made from
    manifest["provenance"] = {"mechanism": "declared-json",
                              "inputs": {"tu": hashlib.sha256(source.read_bytes()).hexdigest(),
                                         "manifest": hashlib.sha256(manifest_path.read_bytes()).hexdigest()}}
    data = container.pack(manifest, payload)
    out = Path(out) if out else source.with_suffix(".plink")
    out.write_bytes(data)
    return out
