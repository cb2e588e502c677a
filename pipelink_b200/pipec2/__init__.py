"""pipec2-compatible link driver for sm_100a stage packages.

Re-authored surface of the reference's ``pipec2`` (pipec/src/pipec2): ``.plink`` packages
(zip of ``manifest.json`` + LTO object), provides/needs contract checks between stage
manifests, protocol expansion, a Z3 solve of ring depths and resource bases, generated
binding stub + dispatch kernel, and an nvJitLink LTO link into one ``pipeline.cubin`` with a
``link.json`` receipt. Diagnostics carry the reference's clause IDs.
"""
from .model import CLAUSES, LinkResult, PipeLinkError  # noqa: F401
