"""Canonical JSON: sorted keys, ``,``/``:`` separators, one trailing LF
(pipec/src/pipec2/canonjson.py:8-18)."""
import hashlib
import json


def dumps(obj) -> str:
    return json.dumps(obj, sort_keys=True, separators=(",", ":"), ensure_ascii=False) + "\n"


def sha256(obj) -> str:
    return hashlib.sha256(dumps(obj).encode()).hexdigest()
