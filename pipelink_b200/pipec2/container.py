"""``.plink`` = zip with exactly ``manifest.json`` (canonical JSON) and ``stage.o``; DEFLATE 9,
timestamp 1980-01-01, mode 0600 (pipec/src/pipec2/container.py:14-40,80-114)."""
import hashlib
import io
import json
import zipfile

from . import canonjson
from .model import fail

_MEMBERS = ("manifest.json", "stage.o")


def pack(manifest: dict, payload: bytes) -> bytes:
    if "sha256" in manifest.get("payload", {}):
        fail("P-CONTAINER", "payload.sha256", "a source manifest must not carry a payload digest")
    manifest = dict(manifest, payload={"file": "stage.o", "sha256": hashlib.sha256(payload).hexdigest()})
    buf = io.BytesIO()
    with zipfile.ZipFile(buf, "w", zipfile.ZIP_DEFLATED, compresslevel=9) as z:
        for name, data in (("manifest.json", canonjson.dumps(manifest).encode()), ("stage.o", payload)):
            info = zipfile.ZipInfo(name, date_time=(1980, 1, 1, 0, 0, 0))
            info.compress_type = zipfile.ZIP_DEFLATED
            info.external_attr = 0o600 << 16
            z.writestr(info, data, compresslevel=9)
    return buf.getvalue()


def read(path_or_bytes):
    data = path_or_bytes if isinstance(path_or_bytes, bytes) else open(path_or_bytes, "rb").read()
    try:
        with zipfile.ZipFile(io.BytesIO(data)) as z:
            names = tuple(z.namelist())
            if names != _MEMBERS:
                fail("P-CONTAINER", "members", f"expected {_MEMBERS}, found {names}")
            manifest = json.loads(z.read("manifest.json"))
            payload = z.read("stage.o")
    except zipfile.BadZipFile as exc:
        fail("P-CONTAINER", "zip", str(exc))
    if hashlib.sha256(payload).hexdigest() != manifest.get("payload", {}).get("sha256"):
        fail("P-CONTAINER", "payload.sha256", "payload digest does not match the manifest")
    return manifest, payload
