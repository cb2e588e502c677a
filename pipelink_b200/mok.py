"""Host side of the MXFP8 MoE forward path (single rank or one rank of an expert-parallel group).

Mirrors the reference's session object ``MoKHost`` (campaigns/mok/host/mok_port_host.py:72-239):
same ``Shape`` / ``Inputs`` records, the same step order for ``forward`` (schedule -> dispatch ->
gate/up GEMM + SwiGLU -> down GEMM + combine placement -> weighted epilogue), the same names for
the forward-context tensors it returns, and ``ops.mxfp8_quantize`` for weights. All device work
goes through the C ABI in ``include/pipelink_b200.h``; torch only owns the memory and the stream.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib

def expert_padding() -> int:
    """Rows every expert segment is padded to: one grouped-GEMM tile (256, as in the reference,
    campaigns/mok/port/framework/interp_fwd.cu:324)."""
    return _lib.load().plb_moe_tile_rows()


@dataclass(frozen=True)
class Shape:
    name: str
    experts: int
    hidden: int
    intermediate: int
    topk: int
    tokens: int


SANITY = Shape("sanity", 4, 256, 256, 1, 512)
CONFIG2 = Shape("moe-ffn-fwd", 64, 4096, 2048, 8, 16384)


@dataclass(frozen=True)
class Inputs:
    x: torch.Tensor        # bf16 [tokens, hidden]
    experts: torch.Tensor  # int [tokens, topk]
    router: torch.Tensor   # fp32 [tokens, topk]


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def schedule_capacity(tokens_total: int, num_local_experts: int, padding: int | None = None) -> int:
    """Rows that always suffice: every routed row plus worst-case padding, rounded to a tile."""
    padding = padding or expert_padding()
    need = tokens_total + num_local_experts * (padding - 1)
    return (need + padding - 1) // padding * padding


def mxfp8_quantize(t: torch.Tensor, normal: bool = True, transposed: bool = False, live_rows: torch.Tensor | None = None):
    """``ops.mxfp8_quantize(tensor, normal, transposed)`` (mok_port_host.py:122).

    ``t`` is bf16 ``[..., rows, cols]`` on the device; leading dims are folded into rows.
    Returns ``(fp8, sc, fp8_t, sc_t)`` with ``None`` for the orientation not requested; fp8
    tensors are uint8, scales are uint8 ``[rows/128, cols/128, 32, 16]``. ``live_rows`` (a device
    int32 scalar, the schedule's row count): only the 128-row tiles below it are read and written,
    for routed buffers that are sized for the worst case.
    """
    if t.dtype != torch.bfloat16 or not t.is_cuda or not t.is_contiguous():
        raise ValueError("mxfp8_quantize wants a contiguous CUDA bf16 tensor")
    cols = t.shape[-1]
    rows = t.numel() // cols
    if rows % 128 or cols % 128:
        raise ValueError("rows and cols must be multiples of 128")
    dev = t.device
    q = sc = qt = sct = None
    if normal:
        q = torch.empty(t.shape, dtype=torch.uint8, device=dev)
        sc = torch.empty((rows // 128, cols // 128, 32, 16), dtype=torch.uint8, device=dev)
    if transposed:
        if t.dim() != 2:
            raise ValueError("the transposed orientation is defined for 2-D tensors")
        qt = torch.empty((cols, rows), dtype=torch.uint8, device=dev)
        sct = torch.empty((cols // 128, rows // 128, 32, 16), dtype=torch.uint8, device=dev)
    _lib.call("plb_mxfp8_quantize_live", t.data_ptr(), rows, cols, _ptr(live_rows), _ptr(q), _ptr(sc), _ptr(qt),
              _ptr(sct), _stream())
    return q, sc, qt, sct


def mxfp8_dequantize(q: torch.Tensor, sc: torch.Tensor) -> torch.Tensor:
    cols = q.shape[-1]
    rows = q.numel() // cols
    out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    _lib.call("plb_mxfp8_dequantize", q.data_ptr(), sc.data_ptr(), rows, cols, out.data_ptr(),
              _stream())
    return out


class DeviceStatus:
    """The 32-byte status record the kernels write on a bounded-wait failure."""

    def __init__(self, device):
        self.buf = torch.zeros(8, dtype=torch.int32, device=device)

    def reset(self):
        self.buf.zero_()

    def check(self, where: str = ""):
        """Synchronises, then raises if a kernel recorded a failure."""
        vals = self.buf.cpu().tolist()
        if vals[0] != 0:
            name = _lib.STATUS_NAMES.get(vals[0], "unknown")
            raise RuntimeError(f"device status {vals[0]} ({name}) {where}: cta={vals[1]} what={vals[2]} "
                               f"observed={vals[3] & 0xFFFFFFFF} expected={vals[4] & 0xFFFFFFFF}")


class Schedule:
    """Device arrays written by ``plb_moe_schedule`` (fields of upstream's schedule object)."""

    def __init__(self, world, tokens, topk, num_local_experts, capacity, device):
        i32 = dict(dtype=torch.int32, device=device)
        self.capacity = capacity
        self.peer_rank = torch.empty(capacity, **i32)
        self.peer_token_idx = torch.empty(capacity, **i32)
        self.dest_row = torch.empty(capacity, **i32)
        self.num_tokens = torch.zeros(1, **i32)
        self.tokens_per_expert = torch.zeros(num_local_experts, **i32)
        self.expert_offsets = torch.zeros(num_local_experts + 1, **i32)
        self.block_expert = torch.empty(capacity // 128, **i32)
        nbytes = _lib.load().plb_moe_schedule_scratch_bytes(world, tokens, topk, num_local_experts)
        self.scratch = torch.empty(max(nbytes, 4) // 4, **i32)


class MoKHost:
    """One rank's persistent forward session."""

    def __init__(self, shape: Shape, *, device="cuda", rank: int = 0, world: int = 1,
                 padding: int | None = None, capacity: int | None = None, swiglu_limit: float = 0.0,
                 precision: str = "mxfp8"):
        if precision not in ("mxfp8", "bf16"):
            raise ValueError("precision is 'mxfp8' or 'bf16'")
        if shape.experts % world:
            raise ValueError("shape/process group disagrees: experts % world != 0")
        _lib.load()
        padding = padding or expert_padding()
        if shape.hidden % expert_padding() or shape.intermediate % expert_padding():
            raise ValueError(f"hidden and intermediate must be multiples of {expert_padding()}")
        self.shape, self.rank, self.world, self.padding = shape, rank, world, padding
        # clamped-SwiGLU variant of this session (the reference's c1 cells use 4.0,
        # campaigns/mok/README.md:82-84); applied to the library before each activation launch
        self.swiglu_limit = float(swiglu_limit)
        # routed precision of this session (pipelink_mok_precision of the reference's links,
        # campaigns/mok/README.md:86-93): "bf16" runs every grouped GEMM on bf16 operands
        self.precision = precision
        self.pull_variant = "loads"     # dispatch pull: "loads" (16-byte loads per lane) or "bulk" (bulk-copy engine)
        self.device = torch.device(device)
        E = shape.experts // world
        L, H, I, k = shape.tokens, shape.hidden, shape.intermediate, shape.topk
        self.num_local_experts = E
        self.capacity = capacity or schedule_capacity(world * L * k, E, padding)
        P = self.capacity
        u8 = dict(dtype=torch.uint8, device=self.device)
        self.status = DeviceStatus(self.device)
        self.schedule = Schedule(world, L, k, E, P, self.device)
        self.routes_i32 = torch.empty((world, L, k), dtype=torch.int32, device=self.device)
        # tokens are quantised once at home (rows padded to a whole 128-row scale block), then
        # dispatch gathers E4M3 rows + scale words; identical bytes to quantising gathered rows
        L_pad = (L + 127) // 128 * 128
        self._x_storage = torch.zeros((L_pad, H), dtype=torch.bfloat16, device=self.device)
        self.x_buffer = self._x_storage[:L]
        self.router_weight_buffer = torch.empty((L, k), dtype=torch.float32, device=self.device)
        self.xq = torch.empty((L_pad, H), **u8)
        self.xsc = torch.empty((L_pad // 128, H // 128, 32, 16), **u8)
        self.xq_peers = torch.tensor([self.xq.data_ptr()] * world, dtype=torch.int64, device=self.device)
        self.xsc_peers = torch.tensor([self.xsc.data_ptr()] * world, dtype=torch.int64, device=self.device)
        # the same scale words with one contiguous run per token (what the bulk-copy dispatch fetches)
        self.xsc_rows = torch.empty((L_pad, H // 128), dtype=torch.int32, device=self.device)
        self.xsc_rows_peers = torch.tensor([self.xsc_rows.data_ptr()] * world, dtype=torch.int64, device=self.device)
        self.dispatch_scratch = torch.zeros(P // 256 + 1, dtype=torch.int32, device=self.device)
        # dispatch inside the gate/up GEMM kernel instead of a pull kernel in front of it
        self.fused_dispatch = False
        self.buffers = {
            "x_routed_fp8": torch.empty((P, H), **u8),
            "x_routed_sc": torch.empty((P // 128, H // 128, 32, 16), **u8),
            "hidden_routed_fp8": torch.empty((P, I), **u8),
            "hidden_routed_sc": torch.empty((P // 128, I // 128, 32, 16), **u8),
            "combine_buffer": torch.empty((L * k, H), dtype=torch.bfloat16, device=self.device),
            "output": torch.empty((L, H), dtype=torch.bfloat16, device=self.device),
        }
        if precision == "bf16":
            bf = dict(dtype=torch.bfloat16, device=self.device)
            self.buffers.update(x_routed_bf16=torch.empty((P, H), **bf), hidden_routed_bf16=torch.empty((P, I), **bf))
        self.weights = None

    # ------------------------------------------------------------------ weights
    def load_weights(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                     keep_unpacked: bool = True, train: bool = False):
        """bf16 [E, I, H], [E, I, H], [E, H, I] for this rank's experts. ``train=True`` also
        prepares the transposed-quantised weights the data gradients contract with
        (``w_routed_*_t`` of campaigns/mok/host/resources.py:75-77)."""
        E, I, H = self.num_local_experts, self.shape.intermediate, self.shape.hidden
        if tuple(w_gate.shape) != (E, I, H) or tuple(w_up.shape) != (E, I, H) or tuple(w_down.shape) != (E, H, I):
            raise ValueError("weight shapes disagree with the session shape")
        if self.precision == "bf16":
            # per 256 rows of the gate/up operand: 128 gate rows, then the 128 up rows of the same columns
            w13 = torch.stack([w_gate.reshape(E, I // 128, 128, H), w_up.reshape(E, I // 128, 128, H)], dim=2)
            self.weights = dict(w13_bf16=w13.reshape(E, 2 * I, H).to(torch.bfloat16).contiguous(),
                                w_routed_down_bf16=w_down.to(torch.bfloat16).contiguous())
            if train:
                # the data gradients contract with the transposed weights: W_down^T [E, I, H], [W_gate; W_up]^T [E, H, 2I]
                self.weights.update(
                    w_down_t_bf16=w_down.to(torch.bfloat16).transpose(1, 2).contiguous(),
                    w_cat_t_bf16=torch.cat([w_gate, w_up], dim=1).to(torch.bfloat16).transpose(1, 2).contiguous())
                self._alloc_train_buffers()
            return
        gq, gsc, _, _ = mxfp8_quantize(w_gate.contiguous())
        uq, usc, _, _ = mxfp8_quantize(w_up.contiguous())
        dq, dsc, _, _ = mxfp8_quantize(w_down.contiguous())
        self.load_quantized_weights(gq, gsc, uq, usc, dq, dsc, keep_unpacked=keep_unpacked)
        if train:
            u8 = dict(dtype=torch.uint8, device=self.device)
            wdt = torch.empty((E, I, H), **u8)                       # W_down^T, blocks along H
            wdt_sc = torch.empty((E * I // 128, H // 128, 32, 16), **u8)
            wct = torch.empty((E, H, 2 * I), **u8)                   # [W_gate; W_up]^T, blocks along 2I
            wct_sc = torch.empty((E * H // 128, 2 * I // 128, 32, 16), **u8)
            for e in range(E):
                _, _, t, tsc = mxfp8_quantize(w_down[e].contiguous(), False, True)
                wdt[e].copy_(t)
                wdt_sc[e * I // 128:(e + 1) * I // 128].copy_(tsc)
                _, _, t, tsc = mxfp8_quantize(torch.cat([w_gate[e], w_up[e]]).contiguous(), False, True)
                wct[e].copy_(t)
                wct_sc[e * H // 128:(e + 1) * H // 128].copy_(tsc)
            self.weights.update(w_down_t_fp8=wdt, w_down_t_sc=wdt_sc, w_cat_t_fp8=wct, w_cat_t_sc=wct_sc)
            self._alloc_train_buffers()

    def load_quantized_weights(self, gq, gsc, uq, usc, dq, dsc, keep_unpacked: bool = True):
        E, I, H = self.num_local_experts, self.shape.intermediate, self.shape.hidden
        w13 = torch.empty((E, 2 * I, H), dtype=torch.uint8, device=self.device)
        w13_sc = torch.empty((E * 2 * I // 128, H // 128, 32, 16), dtype=torch.uint8, device=self.device)
        _lib.call("plb_moe_pack_gate_up", gq.data_ptr(), gsc.data_ptr(), uq.data_ptr(), usc.data_ptr(),
                  E, I, H, w13.data_ptr(), w13_sc.data_ptr(), _stream())
        torch.cuda.current_stream().synchronize()
        self.weights = dict(w13_fp8=w13, w13_sc=w13_sc, w_routed_down_fp8=dq, w_routed_down_sc=dsc)
        if keep_unpacked:
            self.weights.update(w_routed_gate_fp8=gq, w_routed_gate_sc=gsc, w_routed_up_fp8=uq,
                                w_routed_up_sc=usc)

    # ------------------------------------------------------------------ steps
    def schedule_into(self, routes_all_ranks: torch.Tensor):
        """routes: int [world, tokens, topk] (already gathered over the group)."""
        s, sh = self.schedule, self.shape
        self.routes_i32.copy_(routes_all_ranks.reshape(self.routes_i32.shape))
        _lib.call("plb_moe_schedule", self.routes_i32.data_ptr(), self.world, sh.tokens, sh.topk,
                  self.rank * self.num_local_experts, self.num_local_experts, self.capacity,
                  self.padding, s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(),
                  s.dest_row.data_ptr(), s.num_tokens.data_ptr(), s.tokens_per_expert.data_ptr(),
                  s.expert_offsets.data_ptr(), s.block_expert.data_ptr(), s.scratch.data_ptr(),
                  s.scratch.numel() * 4, self.status.buf.data_ptr(), _stream())
        return s

    def quantize_tokens(self):
        """x_buffer (bf16) -> xq / xsc, the buffers dispatch pulls rows from."""
        if self.precision == "bf16":
            return                      # rows are gathered as bf16
        rows = self._x_storage.shape[0]
        _lib.call("plb_mxfp8_quantize", self._x_storage.data_ptr(), rows, self.shape.hidden,
                  self.xq.data_ptr(), self.xsc.data_ptr(), None, None, _stream())
        if self.pull_variant == "bulk" or self.fused_dispatch:
            _lib.call("plb_ep_scale_rows", self.xsc.data_ptr(), rows, self.shape.hidden, self.xsc_rows.data_ptr(), _stream())

    def pull(self):
        """Dispatch: gather every scheduled row's E4M3 bytes and scale words (comm.cu:105-123)."""
        if self.precision == "bf16":
            return self.pull_bf16()
        if self.fused_dispatch:
            return                      # the gate/up GEMM kernel pulls its own rows
        self.pull_now()

    def pull_now(self):
        s, b, sh = self.schedule, self.buffers, self.shape
        if self.pull_variant == "bulk" and sh.hidden <= 4096:
            _lib.call("plb_ep_pull_rows_bulk", self.xq_peers.data_ptr(), self.xsc_rows_peers.data_ptr(),
                      s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(), s.num_tokens.data_ptr(),
                      self.capacity, sh.hidden, b["x_routed_fp8"].data_ptr(), b["x_routed_sc"].data_ptr(),
                      1, self.status.buf.data_ptr(), _stream())
            return
        _lib.call("plb_ep_pull_rows", self.xq_peers.data_ptr(), self.xsc_peers.data_ptr(),
                  s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(), s.num_tokens.data_ptr(),
                  self.capacity, sh.hidden, b["x_routed_fp8"].data_ptr(), b["x_routed_sc"].data_ptr(),
                  _stream())

    def pull_bf16(self):
        s, b, sh = self.schedule, self.buffers, self.shape
        _lib.call("plb_moe_gather_rows", self.x_buffer.data_ptr(), s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(),
                  s.num_tokens.data_ptr(), self.capacity, sh.hidden, b["x_routed_bf16"].data_ptr(), _stream())

    def dispatch(self):
        self.quantize_tokens()
        self.pull()

    def select_activation(self):
        _lib.call("plb_moe_set_swiglu_limit", self.swiglu_limit)

    def gemm_gate_up(self):
        s, b, w, sh = self.schedule, self.buffers, self.weights, self.shape
        self.select_activation()
        if self.precision == "bf16":
            _lib.call("plb_moe_gemm_gate_up_bf16", b["x_routed_bf16"].data_ptr(), w["w13_bf16"].data_ptr(),
                      s.block_expert.data_ptr(), s.num_tokens.data_ptr(), self.capacity, self.num_local_experts,
                      sh.intermediate, sh.hidden, b["hidden_routed_bf16"].data_ptr(), self.status.buf.data_ptr(), _stream())
            return
        if self.fused_dispatch:
            _lib.call("plb_moe_gemm_gate_up_dispatch", self.xq_peers.data_ptr(), self.xsc_rows_peers.data_ptr(),
                      s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(), b["x_routed_fp8"].data_ptr(),
                      b["x_routed_sc"].data_ptr(), w["w13_fp8"].data_ptr(), w["w13_sc"].data_ptr(),
                      s.block_expert.data_ptr(), s.num_tokens.data_ptr(), self.capacity, self.num_local_experts,
                      sh.intermediate, sh.hidden, b["hidden_routed_fp8"].data_ptr(), b["hidden_routed_sc"].data_ptr(),
                      self.dispatch_scratch.data_ptr(), self.status.buf.data_ptr(), _stream())
            return
        _lib.call("plb_moe_gemm_gate_up", b["x_routed_fp8"].data_ptr(), b["x_routed_sc"].data_ptr(),
                  w["w13_fp8"].data_ptr(), w["w13_sc"].data_ptr(), s.block_expert.data_ptr(),
                  s.num_tokens.data_ptr(), self.capacity, self.num_local_experts, sh.intermediate,
                  sh.hidden, b["hidden_routed_fp8"].data_ptr(), b["hidden_routed_sc"].data_ptr(),
                  self.status.buf.data_ptr(), _stream())

    def gemm_down(self):
        s, b, w, sh = self.schedule, self.buffers, self.weights, self.shape
        if self.precision == "bf16":
            _lib.call("plb_moe_gemm_down_bf16", b["hidden_routed_bf16"].data_ptr(), w["w_routed_down_bf16"].data_ptr(),
                      s.block_expert.data_ptr(), s.num_tokens.data_ptr(), s.dest_row.data_ptr(), None, self.capacity,
                      self.num_local_experts, sh.intermediate, sh.hidden, 0, b["combine_buffer"].data_ptr(), None,
                      self.status.buf.data_ptr(), _stream())
            return
        _lib.call("plb_moe_gemm_down", b["hidden_routed_fp8"].data_ptr(),
                  b["hidden_routed_sc"].data_ptr(), w["w_routed_down_fp8"].data_ptr(),
                  w["w_routed_down_sc"].data_ptr(), s.block_expert.data_ptr(),
                  s.num_tokens.data_ptr(), s.dest_row.data_ptr(), self.capacity,
                  self.num_local_experts, sh.intermediate, sh.hidden,
                  b["combine_buffer"].data_ptr(), self.status.buf.data_ptr(), _stream())

    def fwd_epilogue(self, y_shared=None):
        b, sh = self.buffers, self.shape
        _lib.call("plb_moe_fwd_epilogue", _ptr(y_shared), b["combine_buffer"].data_ptr(),
                  self.router_weight_buffer.data_ptr(), sh.tokens, sh.topk, sh.hidden,
                  b["output"].data_ptr(), _stream())
        return b["output"]

    # ------------------------------------------------------------------ training
    def _alloc_train_buffers(self):
        P, sh, dev = self.capacity, self.shape, self.device
        H, I, E, k, L = sh.hidden, sh.intermediate, self.num_local_experts, sh.topk, sh.tokens
        u8 = dict(dtype=torch.uint8, device=dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        sc = lambda r, c: torch.empty((r // 128, c // 128, 32, 16), **u8)
        b = self.buffers
        if self.precision == "bf16":
            b.update(gate_routed_bf16=torch.zeros((P, I), **bf), up_routed_bf16=torch.zeros((P, I), **bf),
                     d_y_routed=torch.zeros((P, H), **bf), d_hidden_routed=torch.zeros((P, I), **bf),
                     d_gate_up_routed=torch.zeros((P, 2 * I), **bf),
                     d_x_routed_buffer=torch.zeros((L * k, H), **bf), d_x=torch.empty((L, H), **bf),
                     d_router_weights=torch.zeros((L, k), dtype=torch.float32, device=dev),
                     d_w_routed_down=torch.empty((E, H, I), **bf), d_w_routed_gate_up=torch.empty((E, 2 * I, H), **bf),
                     # transposes of the row-major activations: the operands of the weight-gradient GEMMs
                     t_rows_h=torch.zeros((H, P), **bf), t_rows_i=torch.zeros((I, P), **bf),
                     t_rows_2i=torch.zeros((2 * I, P), **bf), t_rows_h2=torch.zeros((H, P), **bf))
            b["x_routed_bf16"].zero_()
            b["hidden_routed_bf16"].zero_()
            self._ones = torch.ones((L, k), dtype=torch.float32, device=dev)
            self._identity_rows = torch.arange(P, dtype=torch.int32, device=dev)
            return
        b.update(gate_routed_fp8=torch.empty((P, I), **u8), gate_routed_sc=sc(P, I),
                 up_routed_fp8=torch.empty((P, I), **u8), up_routed_sc=sc(P, I),
                 hidden_routed_bf16=torch.zeros((P, I), **bf),
                 d_y_routed=torch.empty((P, H), **bf), d_hidden_routed=torch.zeros((P, I), **bf),
                 d_gate_up_routed=torch.empty((P, 2 * I), **bf), x_routed_bf16=torch.empty((P, H), **bf),
                 d_x_routed_buffer=torch.zeros((L * k, H), **bf), d_x=torch.empty((L, H), **bf),
                 d_router_weights=torch.zeros((L, k), dtype=torch.float32, device=dev),
                 d_w_routed_down=torch.empty((E, H, I), **bf), d_w_routed_gate_up=torch.empty((E, 2 * I, H), **bf))
        self._ones = torch.ones((L, k), dtype=torch.float32, device=dev)
        self._identity_rows = torch.arange(P, dtype=torch.int32, device=dev)

    def gemm_gate_up_train(self):
        s, b, w, sh = self.schedule, self.buffers, self.weights, self.shape
        self.select_activation()
        if self.precision == "bf16":
            _lib.call("plb_moe_gemm_gate_up_bf16_train", b["x_routed_bf16"].data_ptr(), w["w13_bf16"].data_ptr(),
                      s.block_expert.data_ptr(), s.num_tokens.data_ptr(), self.capacity, self.num_local_experts,
                      sh.intermediate, sh.hidden, b["hidden_routed_bf16"].data_ptr(), b["gate_routed_bf16"].data_ptr(),
                      b["up_routed_bf16"].data_ptr(), self.status.buf.data_ptr(), _stream())
            return
        if self.fused_dispatch:
            _lib.call("plb_moe_gemm_gate_up_train_dispatch", self.xq_peers.data_ptr(), self.xsc_rows_peers.data_ptr(),
                      s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(), b["x_routed_fp8"].data_ptr(),
                      b["x_routed_sc"].data_ptr(), w["w13_fp8"].data_ptr(), w["w13_sc"].data_ptr(),
                      s.block_expert.data_ptr(), s.num_tokens.data_ptr(), self.capacity, self.num_local_experts,
                      sh.intermediate, sh.hidden, b["hidden_routed_fp8"].data_ptr(), b["hidden_routed_sc"].data_ptr(),
                      b["gate_routed_fp8"].data_ptr(), b["gate_routed_sc"].data_ptr(), b["up_routed_fp8"].data_ptr(),
                      b["up_routed_sc"].data_ptr(), b["hidden_routed_bf16"].data_ptr(), self.dispatch_scratch.data_ptr(),
                      self.status.buf.data_ptr(), _stream())
            return
        _lib.call("plb_moe_gemm_gate_up_train", b["x_routed_fp8"].data_ptr(), b["x_routed_sc"].data_ptr(),
                  w["w13_fp8"].data_ptr(), w["w13_sc"].data_ptr(), s.block_expert.data_ptr(), s.num_tokens.data_ptr(),
                  self.capacity, self.num_local_experts, sh.intermediate, sh.hidden,
                  b["hidden_routed_fp8"].data_ptr(), b["hidden_routed_sc"].data_ptr(),
                  b["gate_routed_fp8"].data_ptr(), b["gate_routed_sc"].data_ptr(),
                  b["up_routed_fp8"].data_ptr(), b["up_routed_sc"].data_ptr(),
                  b["hidden_routed_bf16"].data_ptr(), self.status.buf.data_ptr(), _stream())

    def _gemm_rows(self, a_q, a_sc, b_q, b_sc, K, N, out, dest_rows):
        """bf16 out[dest_rows[p]] = A_q[p] . B_q[expert(p)]^T: plb_moe_gemm_down with K and N named freely."""
        s = self.schedule
        _lib.call("plb_moe_gemm_down", a_q.data_ptr(), a_sc.data_ptr(), b_q.data_ptr(), b_sc.data_ptr(),
                  s.block_expert.data_ptr(), s.num_tokens.data_ptr(), dest_rows.data_ptr(), self.capacity,
                  self.num_local_experts, K, N, out.data_ptr(), self.status.buf.data_ptr(), _stream())

    def _wgrad(self, a_t, a_t_sc, b_t, b_t_sc, m_rows, n_rows, out):
        _lib.call("plb_moe_gemm_wgrad", a_t.data_ptr(), a_t_sc.data_ptr(), b_t.data_ptr(), b_t_sc.data_ptr(),
                  self.schedule.expert_offsets.data_ptr(), self.capacity, self.num_local_experts, m_rows, n_rows,
                  out.data_ptr(), self.status.buf.data_ptr(), _stream())

    def backward(self, d_out: torch.Tensor, *, check: bool = True, recompute: bool = False):
        """Backward of the last ``forward(train=True)`` (single rank). Returns the gradients the
        reference reports (GRAD_NAMES, mok_port_host.py:29-30, routed part): d_x, d_router_weights,
        d_w_routed_gate / up / down. ``recompute=True`` is the reference's recompute pass
        (campaigns/mok/port/framework/interp_rec.cu): the forward was a plain ``forward(inputs)`` that
        kept only what inference keeps, and the gate / up / hidden activations are produced again
        from the routed tokens before the gradients are taken."""
        s, b, w, sh = self.schedule, self.buffers, self.weights, self.shape
        if recompute:
            if "w_down_t_fp8" not in self.weights and "w_down_t_bf16" not in self.weights:
                raise RuntimeError("load_weights(..., train=True) first")
            self.gemm_gate_up_train()
        if self.precision == "bf16":
            return self._backward_bf16(d_out, check)
        P, H, I, k = self.capacity, sh.hidden, sh.intermediate, sh.topk
        nt = s.num_tokens.data_ptr()
        # combine backward + router-weight gradient
        _lib.call("plb_moe_bwd_dy", d_out.data_ptr(), b["combine_buffer"].data_ptr(), self.router_weight_buffer.data_ptr(),
                  s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(), s.dest_row.data_ptr(), nt, P, H, k,
                  b["d_y_routed"].data_ptr(), b["d_router_weights"].data_ptr(), _stream())
        dy_q, dy_sc, dy_t, dy_t_sc = mxfp8_quantize(b["d_y_routed"], True, True, s.num_tokens)
        # down projection: data gradient, then weight gradient (contraction over each expert's rows)
        self._gemm_rows(dy_q, dy_sc, w["w_down_t_fp8"], w["w_down_t_sc"], H, I, b["d_hidden_routed"], self._identity_rows)
        _, _, h_t, h_t_sc = mxfp8_quantize(b["hidden_routed_bf16"], False, True, s.num_tokens)
        self._wgrad(dy_t, dy_t_sc, h_t, h_t_sc, H, I, b["d_w_routed_down"])
        # SwiGLU
        self.select_activation()
        _lib.call("plb_moe_swiglu_bwd", b["gate_routed_fp8"].data_ptr(), b["gate_routed_sc"].data_ptr(),
                  b["up_routed_fp8"].data_ptr(), b["up_routed_sc"].data_ptr(), b["d_hidden_routed"].data_ptr(), nt, P, I,
                  b["d_gate_up_routed"].data_ptr(), _stream())
        dgu_q, dgu_sc, dgu_t, dgu_t_sc = mxfp8_quantize(b["d_gate_up_routed"], True, True, s.num_tokens)
        # gate/up projections: data gradient scattered to (token, slot) rows, then summed per token
        self._gemm_rows(dgu_q, dgu_sc, w["w_cat_t_fp8"], w["w_cat_t_sc"], 2 * I, H, b["d_x_routed_buffer"], s.dest_row)
        _lib.call("plb_moe_fwd_epilogue", None, b["d_x_routed_buffer"].data_ptr(), self._ones.data_ptr(), sh.tokens, k, H,
                  b["d_x"].data_ptr(), _stream())
        _lib.call("plb_moe_gather_rows", self.x_buffer.data_ptr(), s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(),
                  nt, P, H, b["x_routed_bf16"].data_ptr(), _stream())
        _, _, x_t, x_t_sc = mxfp8_quantize(b["x_routed_bf16"], False, True, s.num_tokens)
        self._wgrad(dgu_t, dgu_t_sc, x_t, x_t_sc, 2 * I, H, b["d_w_routed_gate_up"])
        if check:
            self.status.check("after MoE backward")
        g = b["d_w_routed_gate_up"]
        return {"d_x": b["d_x"], "d_router_weights": b["d_router_weights"], "d_w_routed_gate": g[:, :I],
                "d_w_routed_up": g[:, I:], "d_w_routed_down": b["d_w_routed_down"]}

    def _rows_gemm_bf16(self, a_rows, b_t, K, N, out, dest_rows):
        """bf16 out[dest_rows[p]] = A[p] . B_t[expert(p)]^T with A [P, K] and B_t [E, N, K]."""
        s = self.schedule
        _lib.call("plb_moe_gemm_down_bf16", a_rows.data_ptr(), b_t.data_ptr(), s.block_expert.data_ptr(), s.num_tokens.data_ptr(),
                  dest_rows.data_ptr(), None, self.capacity, self.num_local_experts, K, N, 0, out.data_ptr(), None,
                  self.status.buf.data_ptr(), _stream())

    def _wgrad_bf16(self, a_rows, a_t, b_rows, b_t, out):
        """out[e] = A_e^T . B_e over each expert's rows of the schedule: A [P, M], B [P, N] row-major."""
        P, M, N = self.capacity, a_rows.shape[1], b_rows.shape[1]
        live = self.schedule.num_tokens.data_ptr()       # only the rows in use are transposed
        _lib.call("plb_bf16_transpose_live", a_rows.data_ptr(), P, M, live, a_t.data_ptr(), _stream())
        _lib.call("plb_bf16_transpose_live", b_rows.data_ptr(), P, N, live, b_t.data_ptr(), _stream())
        _lib.call("plb_moe_gemm_wgrad_bf16", a_t.data_ptr(), b_t.data_ptr(), self.schedule.expert_offsets.data_ptr(), P,
                  self.num_local_experts, M, N, out.data_ptr(), self.status.buf.data_ptr(), _stream())

    def _backward_bf16(self, d_out, check):
        """The backward pass of the bf16 routed precision: the MXFP8 pass without its quantisations
        (data gradients on the transposed weights, weight gradients on transposed activations)."""
        s, b, w, sh = self.schedule, self.buffers, self.weights, self.shape
        P, H, I, k = self.capacity, sh.hidden, sh.intermediate, sh.topk
        nt = s.num_tokens.data_ptr()
        _lib.call("plb_moe_bwd_dy", d_out.data_ptr(), b["combine_buffer"].data_ptr(), self.router_weight_buffer.data_ptr(),
                  s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(), s.dest_row.data_ptr(), nt, P, H, k,
                  b["d_y_routed"].data_ptr(), b["d_router_weights"].data_ptr(), _stream())
        self._rows_gemm_bf16(b["d_y_routed"], w["w_down_t_bf16"], H, I, b["d_hidden_routed"], self._identity_rows)
        self._wgrad_bf16(b["d_y_routed"], b["t_rows_h"], b["hidden_routed_bf16"], b["t_rows_i"], b["d_w_routed_down"])
        self.select_activation()
        _lib.call("plb_moe_swiglu_bwd_bf16", b["gate_routed_bf16"].data_ptr(), b["up_routed_bf16"].data_ptr(),
                  b["d_hidden_routed"].data_ptr(), nt, P, I, b["d_gate_up_routed"].data_ptr(), _stream())
        self._rows_gemm_bf16(b["d_gate_up_routed"], w["w_cat_t_bf16"], 2 * I, H, b["d_x_routed_buffer"], s.dest_row)
        _lib.call("plb_moe_fwd_epilogue", None, b["d_x_routed_buffer"].data_ptr(), self._ones.data_ptr(), sh.tokens, k, H,
                  b["d_x"].data_ptr(), _stream())
        # the dispatched bf16 token rows of the forward are still in place
        self._wgrad_bf16(b["d_gate_up_routed"], b["t_rows_2i"], b["x_routed_bf16"], b["t_rows_h2"], b["d_w_routed_gate_up"])
        if check:
            self.status.check("after MoE backward (bf16)")
        g = b["d_w_routed_gate_up"]
        return {"d_x": b["d_x"], "d_router_weights": b["d_router_weights"], "d_w_routed_gate": g[:, :I],
                "d_w_routed_up": g[:, I:], "d_w_routed_down": b["d_w_routed_down"]}

    def megakernel(self):
        """The device part between the barriers of the reference's forward (mok_port_host.py:203)."""
        self.dispatch()
        self.gemm_gate_up()
        self.gemm_down()

    def forward(self, inputs: Inputs, *, check: bool = True, train: bool = False):
        """Single-rank forward: every token of ``inputs`` is local and every expert is local.
        ``train=True`` keeps the forward context ``backward`` needs."""
        if self.world != 1:
            raise ValueError("forward() drives one rank; use pipelink_b200.ep for a group")
        if self.weights is None:
            raise RuntimeError("load_weights() first")
        self.status.reset()
        self.schedule_into(inputs.experts[None])
        self.x_buffer.copy_(inputs.x)
        self.router_weight_buffer.copy_(inputs.router)
        if train:
            if "w_down_t_fp8" not in self.weights and "w_down_t_bf16" not in self.weights:
                raise RuntimeError("load_weights(..., train=True) first")
            self.dispatch()
            self.gemm_gate_up_train()
            self.gemm_down()
        else:
            self.megakernel()
        out = self.fwd_epilogue()
        if check:
            self.status.check("after MoE forward")
        return {"output": out, **self.context_tensors()}

    def host_pipeline(self):
        """A forward loop over HOST buffers (see HostPipeline)."""
        return HostPipeline(self)

    def context_tensors(self):
        b = self.buffers
        if self.precision == "bf16":
            return {"x_routed": b["x_routed_bf16"], "hidden_routed": b["hidden_routed_bf16"],
                    "combine_buffer": b["combine_buffer"]}
        return {"x_routed_data": b["x_routed_fp8"], "x_routed_scale": b["x_routed_sc"],
                "hidden_routed_data": b["hidden_routed_fp8"], "hidden_routed_scale": b["hidden_routed_sc"],
                "combine_buffer": b["combine_buffer"]}

    @staticmethod
    def new_inputs(shape: Shape, generation: int, device, rank: int = 0, world: int = 1) -> Inputs:
        """Seeded inputs with the reference harness's recipe (mok_port_host.py:273-282)."""
        gen = torch.Generator(device=device).manual_seed(1234 + rank + generation * world)
        logits = torch.randn(shape.tokens, shape.experts, generator=gen, device=device)
        values, experts = torch.topk(logits, shape.topk, dim=1)
        if generation % 3 == 0:
            experts.copy_(torch.arange(shape.topk, device=device).expand(shape.tokens, -1))
        x = torch.randn(shape.tokens, shape.hidden, generator=gen, device=device, dtype=torch.bfloat16)
        return Inputs(x, experts, torch.softmax(values.float(), dim=-1))


class HostPipeline:
    """Single-rank forward for callers whose tokens and results live in pinned HOST memory.

    Three streams and two-deep staging: while step i computes, the inputs of step i+1 travel
    host -> device and the result of step i-1 travels device -> host, so a loop runs at the pace
    of the slowest of the three instead of their sum. Every step still moves its own inputs and
    its own result; nothing is cached between steps.

        pipe = host.host_pipeline()
        for x, routes, router, out in batches:      # pinned host tensors
            pipe.submit(x, routes, router, out)
        pipe.drain()                                # every `out` is complete after this
    """

    def __init__(self, host: MoKHost):
        if host.world != 1:
            raise ValueError("HostPipeline drives a single-rank session")
        self.host, dev = host, host.device
        L, H, k = host.shape.tokens, host.shape.hidden, host.shape.topk
        self.copy_in, self.copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.x = [torch.empty((L, H), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.routes = [torch.empty((1, L, k), dtype=torch.int32, device=dev) for _ in range(2)]
        self.router = [torch.empty((L, k), dtype=torch.float32, device=dev) for _ in range(2)]
        self.out = [torch.empty((L, H), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.in_ready = [torch.cuda.Event() for _ in range(2)]      # inputs of a slot have landed
        self.in_free = [torch.cuda.Event() for _ in range(2)]       # compute has consumed a slot's inputs
        self.out_ready = [torch.cuda.Event() for _ in range(2)]     # compute has filled a slot's result
        self.out_free = [torch.cuda.Event() for _ in range(2)]      # a slot's result has left the device
        self.step = 0

    def submit(self, h_x, h_routes, h_router, h_out):
        host, i = self.host, self.step % 2
        compute = torch.cuda.current_stream()
        with torch.cuda.stream(self.copy_in):
            if self.step >= 2:
                self.copy_in.wait_event(self.in_free[i])
            self.x[i].copy_(h_x, non_blocking=True)
            self.routes[i].copy_(h_routes.reshape(self.routes[i].shape), non_blocking=True)
            self.router[i].copy_(h_router, non_blocking=True)
            self.in_ready[i].record(self.copy_in)
        compute.wait_event(self.in_ready[i])
        host.x_buffer.copy_(self.x[i])
        host.router_weight_buffer.copy_(self.router[i])
        host.schedule_into(self.routes[i])
        self.in_free[i].record(compute)
        host.megakernel()
        result = host.fwd_epilogue()
        if self.step >= 2:
            compute.wait_event(self.out_free[i])
        self.out[i].copy_(result)
        self.out_ready[i].record(compute)
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(self.out_ready[i])
            h_out.copy_(self.out[i], non_blocking=True)
            self.out_free[i].record(self.copy_out)
        self.step += 1

    def drain(self):
        self.copy_out.synchronize()
        torch.cuda.current_stream().synchronize()
