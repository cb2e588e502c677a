"""The MoE grouped GEMMs as LINKED images: the packages of ``stages/moe`` (load, MMA, comm and
epilogue owners, packed separately) joined by the link driver into ``pipelink_kernel`` images, and
launched here on the buffers of a ``MoKHost`` session in place of the library's own kernels.

    host = mok.MoKHost(shape); host.load_weights(...)
    linked = LinkedMoE(host)            # loads the three images, builds their parameter blocks
    host.schedule_into(...); host.dispatch()
    linked.gemm_gate_up(); linked.gemm_down(); host.fwd_epilogue()
    # or both projections in ONE launch (pass-2 tiles wait on per-row-tile counters of pass 1):
    linked.forward_ffn(); host.fwd_epilogue()

The stage sources are the library kernel's warp roles with every constant the link decides
(ring depth, shared-memory / barrier / tensor-memory bases, warp numbers, counter slots) read
through ``pipelink_*`` handles, and share its epilogue arithmetic, so a linked pass produces the
bits the library produces. Counterpart of the reference's launch of its linked MoE cells
(campaigns/mok/host/mok_port_host.py:100-118,203: one ``session.launch`` per pass).
"""
from __future__ import annotations

import ctypes
import struct
from pathlib import Path

import torch

from . import _lib, mok
from .pipec2.launcher import Session

OUT_DIR = Path(__file__).resolve().parent / "stages" / "moe" / "out"
COMPOSITIONS = ("gate_up", "gate_up_dispatch", "down", "fwd", "fwd_dispatch", "fwd_full", "fwd_full_dispatch")


def ensure_built() -> Path:
    if not all((OUT_DIR / c / f).exists() for c in COMPOSITIONS for f in ("pipeline.cubin", "one_tu.cubin")):
        from .stages.moe import build
        build.build(OUT_DIR)
    return OUT_DIR


def _operand_map(t: torch.Tensor) -> bytes:
    """[rows, K] u8, box 128 rows x 128 bytes, 128-byte swizzle."""
    rows, k = t.shape[-2] * (t.numel() // (t.shape[-1] * t.shape[-2])), t.shape[-1]
    buf = (ctypes.c_ubyte * 128)()
    _lib.call("plb_tensor_map_2d_u8", buf, t.data_ptr(), rows, k, 128, 128, 1)
    return bytes(buf)


def _scale_map(t: torch.Tensor) -> bytes:
    """[blocks, 128] u32: one row per 512-byte scale block, box = one row."""
    blocks = t.numel() // 512
    buf = (ctypes.c_ubyte * 128)()
    _lib.call("plb_tensor_map_2d_u32", buf, t.data_ptr(), blocks, 128, 1, 128)
    return bytes(buf)


class LinkedMoE:
    def __init__(self, host: mok.MoKHost, out_dir=None, image: str = "pipeline.cubin"):
        """image: "pipeline.cubin" (the linked image) or "one_tu.cubin" (the same sources compiled as
        one translation unit: the control a linked image is timed against)."""
        if host.precision != "mxfp8":
            raise ValueError("the linked images are the MXFP8 GEMMs")
        self.host = host
        out = Path(out_dir or ensure_built())
        self.sessions = {c: Session(out / c, image) for c in COMPOSITIONS}
        slots = self.sessions["gate_up_dispatch"].link["bindings"]
        self.rows_ready_slot, self.ticket_slot = slots["pipelink_moe_rows_ready"][0], slots["pipelink_moe_ticket"][0]
        # the images' counter workspace (gmem_counter domain): zeroed on the stream before a launch that uses it
        self.counters = torch.zeros(2 * 4096 + 64, dtype=torch.int32, device=host.device)
        self.sms = torch.cuda.get_device_properties(host.device).multi_processor_count & ~1
        self.inf = float("inf")

    def _geometry(self, k: int, n_rows: int, rotation: int = 0, stride: int = 1) -> bytes:
        h, s = self.host, self.host.schedule
        return struct.pack("<QQQiiiiii", s.block_expert.data_ptr(), s.num_tokens.data_ptr(), h.status.buf.data_ptr(),
                           h.capacity // 256, k // 128, n_rows // 256, rotation, stride, 0)

    def _launch(self, name: str):
        self.sessions[name].launch((self.sms, 1, 1), torch.cuda.current_stream().cuda_stream)

    def gemm_gate_up(self, dispatch: bool = False):
        """plb_moe_gemm_gate_up (or, with dispatch, plb_moe_gemm_gate_up_dispatch) through a linked image."""
        h, b, w, sh = self.host, self.host.buffers, self.host.weights, self.host.shape
        name = "gate_up_dispatch" if dispatch else "gate_up"
        s = self.sessions[name]
        g = self._geometry(sh.hidden, 2 * sh.intermediate)
        counters = 0
        if dispatch:
            if h.capacity // 256 > 4096 or sh.hidden > 4096:
                raise ValueError("the dispatch image counts at most 4096 row tiles of rows up to 4096 bytes")
            self.counters.zero_()
            counters = self.counters.data_ptr()
            sched = h.schedule
            s.set_params("moe.comm.dispatch", g + struct.pack("<QQQQQQQii", h.xq_peers.data_ptr(), h.xsc_rows_peers.data_ptr(),
                                                              sched.peer_rank.data_ptr(), sched.peer_token_idx.data_ptr(),
                                                              b["x_routed_fp8"].data_ptr(), b["x_routed_sc"].data_ptr(),
                                                              counters, sh.hidden, 0))
        s.set_params("moe.load", _operand_map(b["x_routed_fp8"]) + _operand_map(w["w13_fp8"]) + _scale_map(b["x_routed_sc"]) +
                     _scale_map(w["w13_sc"]) + g + struct.pack("<Q", counters))
        s.set_params("moe.mma", g)
        limit = h.swiglu_limit if h.swiglu_limit > 0 else self.inf
        s.set_params("moe.epilogue.swiglu-mxfp8", g + struct.pack("<QQif", b["hidden_routed_fp8"].data_ptr(),
                                                                   b["hidden_routed_sc"].data_ptr(), sh.intermediate, limit))
        self._launch(name)

    def gemm_down(self, dest_rows=None, out=None, out_peers=None, rotation: int = 0, stride: int = 1):
        """plb_moe_gemm_down (local placement) or, with a device table of per-rank bases,
        plb_moe_gemm_down_push, through the linked image."""
        h, b, w, sh = self.host, self.host.buffers, self.host.weights, self.host.shape
        s = self.sessions["down"]
        g = self._geometry(sh.intermediate, sh.hidden, rotation, stride)
        sched = h.schedule
        dest = sched.dest_row if dest_rows is None else dest_rows
        out = b["combine_buffer"] if out is None else out
        s.set_params("moe.load", _operand_map(b["hidden_routed_fp8"]) + _operand_map(w["w_routed_down_fp8"]) +
                     _scale_map(b["hidden_routed_sc"]) + _scale_map(w["w_routed_down_sc"]) + g + struct.pack("<Q", 0))
        s.set_params("moe.mma", g)
        s.set_params("moe.epilogue.rows-bf16", g + struct.pack("<QQQQii", out.data_ptr(), 0 if out_peers is None else out_peers.data_ptr(),
                                                                dest.data_ptr(), sched.peer_rank.data_ptr(), sh.hidden, 0))
        self._launch("down")

    def forward_ffn(self, dispatch: bool = False, dest_rows=None, out=None, out_peers=None, rotation: int = 0, stride: int = 1,
                    tail=None):
        """Gate/up projection + SwiGLU + requantise, then the down projection with its row placement (or
        combine push), in ONE launch of a linked image: the work of gemm_gate_up() followed by gemm_down().
        With dispatch, the comm owner also pulls the routed rows from the home ranks under the mainloop.
        With `tail` (see forward_full) the same launch ends with the group barrier and the weighted epilogue."""
        h, b, w, sh = self.host, self.host.buffers, self.host.weights, self.host.shape
        name = ("fwd_full" if tail is not None else "fwd") + ("_dispatch" if dispatch else "")
        s = self.sessions[name]
        if h.capacity // 256 > 4096 or sh.hidden > 4096:
            raise ValueError("the forward image counts at most 4096 row tiles of rows up to 4096 bytes")
        g1 = self._geometry(sh.hidden, 2 * sh.intermediate)      # rows in schedule order, as the dispatch warps deliver them
        g2 = self._geometry(sh.intermediate, sh.hidden, rotation, stride)
        self.counters.zero_()
        counters = self.counters.data_ptr()
        sched = h.schedule
        if dispatch:
            s.set_params("moe.comm.dispatch", g1 + struct.pack("<QQQQQQQii", h.xq_peers.data_ptr(), h.xsc_rows_peers.data_ptr(),
                                                               sched.peer_rank.data_ptr(), sched.peer_token_idx.data_ptr(),
                                                               b["x_routed_fp8"].data_ptr(), b["x_routed_sc"].data_ptr(),
                                                               counters, sh.hidden, 0))
        s.set_params("moe.fwd.load",
                     _operand_map(b["x_routed_fp8"]) + _operand_map(w["w13_fp8"]) + _scale_map(b["x_routed_sc"]) +
                     _scale_map(w["w13_sc"]) + _operand_map(b["hidden_routed_fp8"]) + _operand_map(w["w_routed_down_fp8"]) +
                     _scale_map(b["hidden_routed_sc"]) + _scale_map(w["w_routed_down_sc"]) + g1 + g2 +
                     struct.pack("<Qii", counters, 1 if dispatch else 0, 0))
        s.set_params("moe.fwd.mma", g1 + g2)
        dest = sched.dest_row if dest_rows is None else dest_rows
        out = b["combine_buffer"] if out is None else out
        limit = h.swiglu_limit if h.swiglu_limit > 0 else self.inf
        epilogue = g1 + g2 + struct.pack(
            "<QQQQQQQiifi", b["hidden_routed_fp8"].data_ptr(), b["hidden_routed_sc"].data_ptr(), out.data_ptr(),
            0 if out_peers is None else out_peers.data_ptr(), dest.data_ptr(), sched.peer_rank.data_ptr(), counters,
            sh.intermediate, sh.hidden, limit, 0)
        if tail is None:
            s.set_params("moe.fwd.epilogue", epilogue)
        else:
            # MoeFwdCombineParams = {MoeFwdEpilogueParams (176 bytes with its tail padding), MoeFwdTailParams}
            s.set_params("moe.fwd.epilogue.combine", epilogue.ljust(176, b"\0") + tail)
        self._launch(name)

    def forward_full(self, dispatch: bool = False, *, dest_rows=None, out_peers=None, rotation: int = 0, stride: int = 1,
                     combine=None, index=None, flags_peers=None, barrier_state=None, rank: int = 0, world: int = 1):
        """The whole forward after the schedule in ONE launch: forward_ffn() followed, inside the same launch,
        by the group barrier (every rank's rows have landed; one rank: every CTA is done) and the weighted
        epilogue into the session's output. `combine` / `index`: where the epilogue reads a (token, slot)
        row (default: the session's combine buffer at token * topk + slot)."""
        h, b, sh = self.host, self.host.buffers, self.host.shape
        combine = b["combine_buffer"] if combine is None else combine
        tail = struct.pack("<QQQQQQqiiii", combine.data_ptr(), 0 if index is None else index.data_ptr(),
                           h.router_weight_buffer.data_ptr(), b["output"].data_ptr(),
                           0 if flags_peers is None else flags_peers.data_ptr(),
                           0 if barrier_state is None else barrier_state.data_ptr(), sh.tokens, sh.topk, sh.hidden, rank, world)
        self.forward_ffn(dispatch, dest_rows=dest_rows, out_peers=out_peers, rotation=rotation, stride=stride, tail=tail)
        return b["output"]

    def close(self):
        for s in self.sessions.values():
            s.close()
        self.sessions = {}
