"""Clause catalogue, errors and the link receipt (pipec/src/pipec2/model.py:72-101,231-255,840-862)."""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any

CLAUSES = {
    "L-ALIGN": "claim bases satisfy alignment and granularity",
    "L-BUDGET": "resource demands fit the target domains",
    "L-ENTRYABI": "stage entry points use the v2 entry ABI",
    "L-HANDLE": "handle declarations and references are complete and consistent",
    "L-LINK": "device link of the stage payloads and generated units succeeds",
    "L-OVERLAP": "claims with intersecting lifetimes do not overlap",
    "L-OWNER": "every claim and init materializer has exactly one consistent owner",
    "L-PAIR": "every channel has exactly one producer and one consumer endpoint",
    "L-PARAMS": "stage and aggregate parameter layouts satisfy the target ABI",
    "L-PHASE": "claim phases and pairwise exclusions are finite and valid",
    "L-PROTO": "paired endpoint protocols expand consistently",
    "L-REGS": "register choices fit the register file",
    "L-STUB": "generated binding stubs resolve every handle",
    "L-SYM": "symbols are unique and every undefined symbol is resolved",
    "L-TOPO": "stage topology constraints have a legal intersection",
    "L8": "paired endpoints describe the identical physical layout",
    "T-CONTRACT": "a stage's tensor import / export section is well formed",
    "T-MODEL": "a tensor connection stays inside the modelled vocabulary",
    "T-PLAN": "a route for the tensor connection is certified within the import's lends",
    "T-PLAN-RENDEZVOUS": "a tensor import declares its outer ready and done events",
    "T-PLAN-FRAME": "a register export is given one frame lend with enough positions",
    "T-LOWER": "the certified program lowers to an adapter for the site it runs at",
    "P-ANNOTATION": "a unit's annotations state exactly one stage, one parameter block and at most one topology",
    "P-COMPILE": "the stage payload compiles for the target profile",
    "P-INIT": "a barrier ring's declared initialising warp belongs to its owner role",
    "P-CONTAINER": "the package container is well formed",
    "P-SYM": "stage symbols carry the stage's symbol prefix",
}


@dataclass(frozen=True)
class ClauseFailure:
    clause_id: str
    path: str
    message: str
    detail: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.clause_id not in CLAUSES:
            raise ValueError(f"unknown clause ID {self.clause_id!r}")


class PipeLinkError(RuntimeError):
    """Deterministic link/pack failure: ``[CLAUSE] path: message`` for every failure."""

    def __init__(self, failures):
        if isinstance(failures, ClauseFailure):
            failures = [failures]
        self.failures = sorted(failures, key=lambda f: (f.clause_id, f.path))
        super().__init__("; ".join(f"[{f.clause_id}] {f.path}: {f.message}" for f in self.failures))


def fail(clause, path, message, **detail):
    raise PipeLinkError(ClauseFailure(clause, path, message, detail))


@dataclass
class LinkResult:
    kernel_symbol: str
    threads: int
    regs_cap: int
    dyn_smem_bytes: int
    cluster: tuple
    params: dict                      # {total_bytes, align, entries [[stage, offset, bytes, align]]}
    bindings: dict                    # handle -> [value, "solved" | "forced"]
    variants: dict
    intervals: dict                   # domain -> [{handle, lo, hi, phase}]
    protocol_expansions: list
    observed: tuple                   # (registers, stack, local) of the linked kernel, -1 if unknown
    input_hashes: dict
    generated_hashes: dict
    sass_report: Any = None
    solver: dict | None = None
    roles: list | None = None         # [{stage, role, entry, warp_lo, warp_hi, params_offset}]
    tmem_columns: int = 0
    tensor: list | None = None        # one record per tensor connection: routes tried, certified program, reservations

    def to_json_obj(self):
        return asdict(self)

    @classmethod
    def from_json_obj(cls, obj):
        return cls(**obj)
