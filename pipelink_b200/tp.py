"""Tensor-parallel GEMM compositions of the reference's examples/comm-overlap on the bf16 CTA-pair
GEMM: AllGather -> GEMM (`ag`) and GEMM -> ReduceScatter (`rs`).

    ag:  C_r = gather(A_q) @ B_r^T                       A_q [M/W, K], B_r [N/W, K]  ->  C_r [M, N/W]
    rs:  out_r = (sum_q A_q @ B_q^T)[r*M/W:(r+1)*M/W]    A_q [M, K/W], B_q [N, K/W]  ->  out_r [M/W, N]

(examples/comm-overlap/README.md, "Compositions and ownership"). Peer memory is one symmetric slab
per rank, as on the expert-parallel path (`ep.IpcSlab`, or plain allocations for ranks emulated on
one GPU).

ag: a rank's shard lives in its own gathered buffer; `plb_tp_push_rows` copies it to every peer and
advances per-256-row-block counters there; the GEMM's load lane waits for a block's counter before
its first TMA read of that block and walks the row tiles starting at its own shard, so the peers'
rows arrive while the local ones are multiplied. The gathered buffers and their counters are
double-buffered by step parity, which is all the write-after-read protection the step needs: a rank
can only reach the push of step g+2 after its GEMM of step g+1, which waited for every peer's push
of g+1, which each peer issued after its own GEMM of step g.

rs: the GEMM's epilogue pushes every partial row into the owner's receive slot [row, source rank]
(`plb_tp_gemm_bf16` with `out_peers`), a group barrier publishes the pushes, and the owner sums its
slots in rank order (`plb_moe_fwd_epilogue` on unit weights): two kernels and a barrier, like the
reference's GEMM+push followed by `comm_rs_reduce`, and bitwise repeatable. Slots are double-buffered
by parity. Partials travel as bf16 here (the reference pushes fp32 tiles): results agree with an
fp32 reference to bf16 rounding of W partial sums, not to the reference's 1e-3.
"""
from __future__ import annotations

import torch

from . import _lib
from .ep import barrier_state_for, tensor_from_ptr
from .mok import DeviceStatus, _stream

PARTS = 8            # pieces a 256-row block is pushed in (more CTAs per block, same counter)
TILE = 256


def _align(n: int, a: int = 1024) -> int:
    return (n + a - 1) // a * a


class TpLayout:
    """Byte offsets inside one rank's slab."""

    def __init__(self, m: int, n: int, k: int, world: int):
        if m % (TILE * world) or n % (TILE * world) or k % (128 * world):
            raise ValueError(f"M and N must be multiples of {TILE} * world and K of 128 * world")
        self.m, self.n, self.k, self.world = m, n, k, world
        off = 0
        self.flags = off; off += _align(4 * world)
        self.ready = [0, 0]
        self.gather = [0, 0]
        self.slots = [0, 0]
        for p in range(2):
            self.ready[p] = off; off += _align(4 * (m // TILE))
        for p in range(2):
            self.gather[p] = off; off += _align(m * k * 2)
        for p in range(2):
            self.slots[p] = off; off += _align(m * n * 2)          # [M / W rows, W sources, N]
        self.nbytes = off


class TpRank:
    """One rank's session. ``ptrs[q]`` is rank q's slab as addressable from this process."""

    def __init__(self, layout: TpLayout, rank: int, ptrs, device, distributed: bool):
        _lib.load()
        lay, W = layout, layout.world
        self.layout, self.rank, self.world, self.distributed = lay, rank, W, distributed
        self.device = dev = torch.device(device)
        self.ms, self.nl, self.kl = lay.m // W, lay.n // W, lay.k // W
        i64 = dict(dtype=torch.int64, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        table = lambda off: torch.tensor([p + off for p in ptrs], **i64)
        me = ptrs[rank]
        self.flags_peers = table(lay.flags)
        self.ready_peers = [table(lay.ready[p]) for p in range(2)]
        self.gather_peers = [table(lay.gather[p]) for p in range(2)]
        self.slots_peers = [table(lay.slots[p]) for p in range(2)]
        self.ready = [tensor_from_ptr(me + lay.ready[p], (lay.m // TILE,), torch.int32, dev) for p in range(2)]
        self.gathered = [tensor_from_ptr(me + lay.gather[p], (lay.m, lay.k), torch.bfloat16, dev) for p in range(2)]
        self.slots = [tensor_from_ptr(me + lay.slots[p], (self.ms * W, lay.n), torch.bfloat16, dev) for p in range(2)]
        self.barrier_state = barrier_state_for(me + lay.flags, rank, dev)
        self.status = DeviceStatus(dev)
        # ag and rs advance separately: the gathered buffers and their counters follow the number of
        # ag steps, the receive slots the number of rs steps, whatever order the two are called in
        self.ag_generation = 0
        self.rs_generation = 0
        # helper arrays of the grouped-GEMM entry point: one group, every row live
        self.block_group = torch.zeros(lay.m // 128, **i32)
        self.num_rows = torch.tensor([lay.m], **i32)
        rows = torch.arange(lay.m, **i32)
        self.identity = rows
        self.rs_dest_row = ((rows % self.ms) * W + rank).contiguous()
        self.rs_owner = (rows // self.ms).to(torch.int32).contiguous()
        self.ones = torch.ones((self.ms, W), dtype=torch.float32, device=dev)
        self.rotation = rank * (self.ms // TILE)
        self.ag_out = torch.empty((lay.m, self.nl), dtype=torch.bfloat16, device=dev)
        self.rs_out = torch.empty((self.ms, lay.n), dtype=torch.bfloat16, device=dev)
        self.sms = torch.cuda.get_device_properties(dev).multi_processor_count

    # ------------------------------------------------------------------ all-gather -> GEMM
    def shard_view(self, generation: int | None = None) -> torch.Tensor:
        """Where the caller writes this rank's A shard for the next ``ag`` step ([M/W, K] bf16)."""
        g = self.ag_generation if generation is None else generation
        return self.gathered[g & 1][self.rank * self.ms:(self.rank + 1) * self.ms]

    def ag_push(self):
        p = self.ag_generation & 1
        _lib.call("plb_tp_push_rows", self.shard_view().data_ptr(), self.ms // TILE, TILE * self.layout.k * 2, PARTS,
                  self.rank, self.world, self.gather_peers[p].data_ptr(), self.ready_peers[p].data_ptr(),
                  min(self.sms, (self.ms // TILE) * PARTS * self.world), _stream())

    def ag_gemm(self, b_local: torch.Tensor) -> torch.Tensor:
        lay, p = self.layout, self.ag_generation & 1
        if tuple(b_local.shape) != (self.nl, lay.k) or b_local.dtype != torch.bfloat16 or not b_local.is_contiguous():
            raise ValueError("B_r is a contiguous bf16 [N / W, K]")
        # every ag step with this parity has added PARTS to each block's counter
        target = ((self.ag_generation >> 1) + 1) * PARTS
        _lib.call("plb_tp_gemm_bf16", self.gathered[p].data_ptr(), b_local.data_ptr(), self.block_group.data_ptr(),
                  self.num_rows.data_ptr(), self.identity.data_ptr(), None, lay.m, self.nl, lay.k, self.rotation,
                  self.ready[p].data_ptr(), target, self.ag_out.data_ptr(), None, self.status.buf.data_ptr(), _stream())
        return self.ag_out

    def ag(self, b_local: torch.Tensor) -> torch.Tensor:
        """One step; the shard for it was written through ``shard_view()``. Push first, GEMM second, on
        one stream: the GEMM waits for the peers' pushes, never for a kernel queued behind it here."""
        self.ag_push()
        out = self.ag_gemm(b_local)
        self.ag_generation += 1
        return out

    # ------------------------------------------------------------------ GEMM -> reduce-scatter
    def barrier(self):
        if self.distributed:
            _lib.call("plb_ep_barrier", self.flags_peers.data_ptr(), self.barrier_state.data_ptr(), self.rank, self.world,
                      self.status.buf.data_ptr(), _stream())

    def rs_gemm_push(self, a_local: torch.Tensor, b_local: torch.Tensor):
        lay, p = self.layout, self.rs_generation & 1
        for t, shape in ((a_local, (lay.m, self.kl)), (b_local, (lay.n, self.kl))):
            if tuple(t.shape) != shape or t.dtype != torch.bfloat16 or not t.is_contiguous():
                raise ValueError("A_q is a contiguous bf16 [M, K / W] and B_q [N, K / W]")
        _lib.call("plb_tp_gemm_bf16", a_local.data_ptr(), b_local.data_ptr(), self.block_group.data_ptr(),
                  self.num_rows.data_ptr(), self.rs_dest_row.data_ptr(), self.rs_owner.data_ptr(), lay.m, lay.n, self.kl,
                  self.rotation, None, 0, None, self.slots_peers[p].data_ptr(), self.status.buf.data_ptr(), _stream())

    def rs_reduce(self) -> torch.Tensor:
        p = self.rs_generation & 1
        _lib.call("plb_moe_fwd_epilogue", None, self.slots[p].data_ptr(), self.ones.data_ptr(), self.ms, self.world,
                  self.layout.n, self.rs_out.data_ptr(), _stream())
        return self.rs_out

    def rs(self, a_local: torch.Tensor, b_local: torch.Tensor) -> torch.Tensor:
        self.rs_gemm_push(a_local, b_local)
        self.barrier()                      # every rank's partial rows have landed in my slots
        out = self.rs_reduce()
        self.rs_generation += 1
        return out


class LocalTpGroup:
    """`world` ranks emulated in one process on one GPU: phases run rank after rank, so every
    counter a GEMM waits for has been advanced before that GEMM is launched."""

    def __init__(self, m: int, n: int, k: int, world: int, device="cuda"):
        from .ep import sym_alloc
        self.layout = TpLayout(m, n, k, world)
        self.slabs = [sym_alloc(self.layout.nbytes) for _ in range(world)]
        self.ranks = [TpRank(self.layout, r, self.slabs, device, False) for r in range(world)]

    def ag(self, a_shards, b_locals):
        for r, a in zip(self.ranks, a_shards):
            r.shard_view().copy_(a)
        for r in self.ranks:
            r.ag_push()
        outs = [r.ag_gemm(b) for r, b in zip(self.ranks, b_locals)]
        for r in self.ranks:
            r.ag_generation += 1
            r.status.check("all-gather GEMM")
        return outs

    def rs(self, a_locals, b_locals):
        for r, a, b in zip(self.ranks, a_locals, b_locals):
            r.rs_gemm_push(a, b)
        outs = [r.rs_reduce() for r in self.ranks]
        for r in self.ranks:
            r.rs_generation += 1
            r.status.check("reduce-scatter GEMM")
        return outs

    def close(self):
        torch.cuda.synchronize()
        for p in self.slabs:
            _lib.call("plb_sym_free", p)
        self.slabs = []


class IpcTpGroup:
    """One process per GPU; IPC handles travel through ``torch.distributed`` at set-up only."""

    def __init__(self, m: int, n: int, k: int, rank: int, world: int, device, group=None):
        from .ep import IpcSlab
        self.layout = TpLayout(m, n, k, world)
        self.slab = IpcSlab(self.layout.nbytes, rank, world, group)
        self.rank = TpRank(self.layout, rank, self.slab.ptrs, device, True)

    def close(self):
        self.slab.close()
