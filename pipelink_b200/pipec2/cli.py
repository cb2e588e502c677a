"""``python -m pipelink_b200.pipec2.cli pack|inspect|link|clauses`` (verbs of pipec/src/pipec2/cli.py:193-263).
The flags the reference's examples pass are accepted as they are: ``pack SRC --profile P -o OUT -I DIR -D NAME=VALUE``,
``inspect PKG --json`` (the whole manifest), ``link PIPELINE --out-dir DIR``, ``clauses --json``; a failure prints
``pipec2: [CLAUSE] path: message; ...`` on stderr, the prefix their checkers parse, and exits 1."""
from __future__ import annotations

import argparse
import json
import sys

from . import container, link as linker, pack as packer
from .model import CLAUSES, PipeLinkError


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="pipec2")
    sub = ap.add_subparsers(dest="verb", required=True)
    p = sub.add_parser("pack")
    p.add_argument("source")
    p.add_argument("--manifest")
    p.add_argument("--profile", default="sm_100a")
    p.add_argument("-o", "--output")
    p.add_argument("-I", dest="includes", action="append", default=[])
    p.add_argument("-D", dest="defines", action="append", default=[])
    p.add_argument("--report", help="also write what was packed (stage id, digests) to this file")
    i = sub.add_parser("inspect")
    i.add_argument("package")
    i.add_argument("--json", action="store_true", help="print the whole manifest")
    l = sub.add_parser("link")
    l.add_argument("pipeline")
    l.add_argument("-o", "--output", "--out-dir", dest="output", required=True)
    l.add_argument("--no-device-link", action="store_true")
    c = sub.add_parser("clauses")
    c.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    try:
        if args.verb == "pack":
            out = packer.pack_cu(args.source, args.manifest, args.output, args.profile, args.includes, args.defines)
            if args.report:
                import hashlib
                from pathlib import Path
                manifest, payload = container.read(out)
                Path(args.report).write_text(json.dumps({"package": str(out), "stage": manifest["stage"]["id"],
                                                         "sha256": hashlib.sha256(Path(out).read_bytes()).hexdigest(),
                                                         "payload_bytes": len(payload), "provenance": manifest.get("provenance")}, indent=1) + "\n")
            print(out)
        elif args.verb == "inspect":
            manifest, payload = container.read(args.package)
            if args.json:
                print(json.dumps(manifest, indent=1, sort_keys=True))
                return 0
            print(json.dumps({"stage": manifest["stage"]["id"], "roles": manifest["stage"]["roles"],
                              "endpoints": [(e["name"], e["direction"]) for e in manifest.get("endpoints", [])],
                              "claims": [c["handle"] for c in manifest.get("claims", [])],
                              "payload_bytes": len(payload)}, indent=1))
        elif args.verb == "link":
            r = linker.link(args.pipeline, args.output, device_link=not args.no_device_link)
            print(json.dumps({"kernel_symbol": r.kernel_symbol, "threads": r.threads, "dyn_smem_bytes": r.dyn_smem_bytes,
                              "bindings": r.bindings}, indent=1))
        elif args.json:
            print(json.dumps(dict(sorted(CLAUSES.items())), indent=1))
        else:
            for cid, text in sorted(CLAUSES.items()):
                print(f"{cid}: {text}")
    except PipeLinkError as exc:
        print(f"pipec2: {exc}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
