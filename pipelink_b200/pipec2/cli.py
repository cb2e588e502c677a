"""``python -m pipelink_b200.pipec2.cli pack|inspect|link|clauses`` (verbs of pipec/src/pipec2/cli.py:193-263)."""
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
    i = sub.add_parser("inspect")
    i.add_argument("package")
    l = sub.add_parser("link")
    l.add_argument("pipeline")
    l.add_argument("-o", "--output", required=True)
    l.add_argument("--no-device-link", action="store_true")
    sub.add_parser("clauses")
    args = ap.parse_args(argv)
    try:
        if args.verb == "pack":
            print(packer.pack_cu(args.source, args.manifest, args.output, args.profile, args.includes, args.defines))
        elif args.verb == "inspect":
            manifest, payload = container.read(args.package)
            print(json.dumps({"stage": manifest["stage"]["id"], "roles": manifest["stage"]["roles"],
                              "endpoints": [(e["name"], e["direction"]) for e in manifest.get("endpoints", [])],
                              "claims": [c["handle"] for c in manifest.get("claims", [])],
                              "payload_bytes": len(payload)}, indent=1))
        elif args.verb == "link":
            r = linker.link(args.pipeline, args.output, device_link=not args.no_device_link)
            print(json.dumps({"kernel_symbol": r.kernel_symbol, "threads": r.threads, "dyn_smem_bytes": r.dyn_smem_bytes,
                              "bindings": r.bindings}, indent=1))
        else:
            for cid, text in sorted(CLAUSES.items()):
                print(f"{cid}: {text}")
    except PipeLinkError as exc:
        print(f"pipec2: {exc}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
