"""Target profile: resource domains and limits of sm_100a
(pipec/src/pipec2/profile.py:107-151: same capacities as the reference's sm_103a/sm_100a)."""
from dataclasses import dataclass


@dataclass(frozen=True)
class Domain:
    unit: str
    capacity: object   # int, or "pipeline": the pipeline description states the capacity
    lowest: int
    granularity: int
    physical: str      # domains sharing a physical resource must not overlap each other
    scale: int         # units -> physical units (an mbarrier slot is 16 bytes of shared memory)


SM_100A = {
    "name": "sm_100a", "lto_arch": "lto_100a", "gencode": ("compute_100a", "lto_100a"), "sm": "sm_100a",
    "param_limit_bytes": 32764, "param_align": 64, "max_threads": 1024,
    "domains": {
        "smem": Domain("bytes", 232448, 0, 1, "smem", 1),
        "mbarrier": Domain("16-byte slots", 232448 // 16, 0, 1, "smem", 16),
        "tmem": Domain("columns", 512, 0, 32, "tmem", 1),
        "named_barrier": Domain("IDs", 16, 1, 1, "named_barrier", 1),
        # pages of shared memory whose number and size the pipeline states (`domains.smem_page`:
        # capacity, page_bytes); page p is bytes [p * page_bytes, (p + 1) * page_bytes)
        "smem_page": Domain("pages", "pipeline", 0, 1, "smem", 1),
        "warp": Domain("launch warps", 32, 0, 1, "warp", 1),
        "regs": Domain("per-thread registers", 256, 24, 8, "regs", 1),
        "gmem_counter": Domain("4-byte slots", "pipeline", 0, 1, "gmem_counter", 1),
    },
    # register file of one SM, setmaxnreg granularity, warps per warpgroup, legal CTA groups and
    # the largest cluster (pipec/src/pipec2/profile.py:141-149 gives sm_103a the same caps)
    "caps": {"regs_per_sm": 65536, "reg_alloc_granularity": 8, "regs_min": 24, "regs_max": 255,
             "warpgroup_warps": 4, "cta_group_legal": (1, 2), "max_cluster": (8, 8, 8)},
}
# B300's profile: the same capacities (pipec/src/pipec2/profile.py:141-149). Packages stamped for it are
# checked and solved here like any other; their device link needs a toolkit that knows the architecture.
SM_103A = dict(SM_100A, name="sm_103a", lto_arch="lto_103", gencode=("compute_103a", "lto_103a"), sm="sm_103a")
# Hopper: no tensor memory, no CTA pairs (pipec/src/pipec2/profile.py, SM_90A). Kept so that the reference's Hopper
# packages can be CHECKED and SOLVED by this driver (its `examples/hopper-gemm-split`); nothing is built for it.
SM_90A = dict(SM_100A, name="sm_90a", lto_arch="lto_90a", gencode=("compute_90a", "lto_90a"), sm="sm_90a",
              domains={k: v for k, v in SM_100A["domains"].items() if k != "tmem"},
              caps=dict(SM_100A["caps"], cta_group_legal=(1,)))
PROFILES = {"sm_100a": SM_100A, "sm_103a": SM_103A, "sm_90a": SM_90A}
