"""Expert-parallel MXFP8 MoE forward: one rank per GPU, experts sharded, tokens stay home.

Host-side counterpart of the reference's EP session (campaigns/mok/host/mok_port_host.py:198-205:
build schedule -> copy x / router weights into symmetric buffers -> barrier -> megakernel ->
barrier -> fwd_epilogue) with the collectives replaced by this library's in-kernel peer-memory
stages: every rank quantises its tokens once, publishes its routes into every peer's gather
buffer, peers pull E4M3 rows over NVLink (``plb_ep_pull_rows``), and the down GEMM's epilogue
pushes result rows into the home rank's combine buffer (``plb_moe_gemm_down_push``).
``torch.distributed`` is used only to exchange the CUDA IPC handles of the symmetric slabs.

Two ways to form a group:
  * ``LocalGroup``  - all ranks live in this process on one device (tests on a single GPU;
    phases run rank after rank on one stream, so no flag barrier is needed or launched);
  * ``IpcGroup``    - one process per GPU; slabs are shared through CUDA IPC handles.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, mok


def _align(n, a=256):
    return (n + a - 1) // a * a


class SlabLayout:
    """Offsets of the peer-visible buffers inside one rank's symmetric slab."""

    def __init__(self, shape: mok.Shape, world: int, train: bool = False, stream: bool = False):
        L, H, k = shape.tokens, shape.hidden, shape.topk
        if L % 128:
            raise ValueError("tokens per rank must be a multiple of 128")
        off = 0
        self.flags = off; off += _align(4 * 32)
        self.xq = off; off += _align(L * H)
        self.xsc = off; off += _align(L // 128 * (H // 128) * 512)
        self.xsc_rows = off; off += _align(L * (H // 128) * 4)     # the same words, one contiguous run per token
        self.routes_all = off; off += _align(world * L * k * 4)
        self.combine = off; off += _align(L * k * H * 2)
        self.stream = stream
        if stream:  # receive streams of the combine push: one per source rank, rows in arrival order
            self.recv = off; off += _align(world * L * k * H * 2)
            self.recv_index = off; off += _align(L * k * 4)
        self.train = train
        if train:   # what the backward pass reads from / writes to a token's home rank
            self.x_bf16 = off; off += _align(L * H * 2)        # tokens, for the gate/up weight gradient
            self.d_out = off; off += _align(L * H * 2)         # upstream gradient
            self.router_w = off; off += _align(L * k * 4)      # router weights (d_y = w * d_out)
            self.d_x_rows = off; off += _align(L * k * H * 2)  # input-gradient rows, one per (token, slot)
            if stream:  # receive streams of the input-gradient push (the forward's hold the combine rows
                        # until the router gradient has read them, so the two cannot share a buffer)
                self.d_x_recv = off; off += _align(world * L * k * H * 2)
        self.nbytes = off


class _RawTensor:
    """Expose a raw device pointer to torch through __cuda_array_interface__."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "version": 3, "strides": None}


def tensor_from_ptr(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    if dtype == torch.bfloat16:
        t = torch.as_tensor(_RawTensor(ptr, shape, "<i2"), device=device)
        return t.view(torch.bfloat16)
    typestr = {torch.uint8: "|u1", torch.int32: "<i4", torch.float32: "<f4"}[dtype]
    return torch.as_tensor(_RawTensor(ptr, shape, typestr), device=device)


def barrier_state_for(flags_ptr: int, rank: int, device) -> torch.Tensor:
    """Generation counter of `plb_ep_barrier` for a session opened on a slab whose flag words start at
    ``flags_ptr``. A barrier adds one to word ``rank`` of every rank's flags, this rank's own included,
    so that word counts the barriers this rank has completed on the slab: a session that starts from
    it lines up with flags an earlier session left behind. One session at a time per slab and rank."""
    torch.cuda.synchronize(device)
    return tensor_from_ptr(flags_ptr + 4 * rank, (1,), torch.int32, device).clone()


def sym_alloc(nbytes: int) -> int:
    out = ctypes.c_void_p()
    _lib.call("plb_sym_alloc", nbytes, ctypes.byref(out))
    return out.value


class LocalGroup:
    """`world` ranks emulated in one process: every slab is an allocation on the current device."""

    def __init__(self, shape: mok.Shape, world: int, device, train: bool = False, stream: bool = False):
        self.world, self.device, self.distributed = world, torch.device(device), False
        self.layout = SlabLayout(shape, world, train, stream)
        self.slabs = [sym_alloc(self.layout.nbytes) for _ in range(world)]

    def ptrs_for(self, rank: int):
        return list(self.slabs)

    def close(self):
        for p in self.slabs:
            _lib.call("plb_sym_free", p)
        self.slabs = []


def exchange_handles(handle: bytes, world: int, group=None):
    """Bootstrap step: every rank contributes its 64-byte IPC handle and receives all of them, in
    rank order. The only use of ``torch.distributed`` on the expert-parallel path (any backend)."""
    import torch.distributed as dist
    if len(handle) != 64:
        raise ValueError("a CUDA IPC memory handle is 64 bytes")
    gathered = [None] * world
    dist.all_gather_object(gathered, bytes(handle), group=group)
    if any(h is None or len(h) != 64 for h in gathered):
        raise RuntimeError("a rank did not contribute a handle")
    return gathered


class IpcSlab:
    """One zero-filled device allocation per rank, mapped into every rank through CUDA IPC.
    ``ptrs[r]`` is rank r's slab as addressable from this process (``ptrs[rank]`` is local)."""

    def __init__(self, nbytes: int, rank: int, world: int, group=None):
        import torch.distributed as dist
        self.rank, self.world = rank, world
        self.local = sym_alloc(nbytes)
        handle = (ctypes.c_ubyte * 64)()
        _lib.call("plb_ipc_export", self.local, handle)
        gathered = exchange_handles(bytes(handle), world, group)
        self.ptrs = []
        for r, h in enumerate(gathered):
            if r == rank:
                self.ptrs.append(self.local)
            else:
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                out = ctypes.c_void_p()
                _lib.call("plb_ipc_import", buf, ctypes.byref(out))
                self.ptrs.append(out.value)
        dist.barrier(group=group)

    def close(self):
        torch.cuda.synchronize()
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                _lib.call("plb_ipc_close", p)
        _lib.call("plb_sym_free", self.local)
        self.ptrs = []


class IpcGroup:
    """One process per GPU; handles travel through ``torch.distributed`` (bootstrap only)."""

    def __init__(self, shape: mok.Shape, rank: int, world: int, device, group=None, train: bool = False,
                 stream: bool = False):
        self.world, self.rank, self.device, self.distributed = world, rank, torch.device(device), True
        self.layout = SlabLayout(shape, world, train, stream)
        self.slab = IpcSlab(self.layout.nbytes, rank, world, group)
        self.peer_ptrs = self.slab.ptrs

    def ptrs_for(self, rank: int):
        assert rank == self.rank
        return list(self.peer_ptrs)

    def close(self):
        self.slab.close()
        self.peer_ptrs = []


class EpMoKHost(mok.MoKHost):
    """One rank of the group. ``shape.tokens`` is tokens per rank, ``shape.experts`` the global count."""

    def __init__(self, shape: mok.Shape, rank: int, group, padding: int | None = None, swiglu_limit: float = 0.0,
                 precision: str = "mxfp8"):
        if precision == "bf16" and not group.layout.train:
            raise ValueError("the bf16 routed precision dispatches bf16 rows: open the group with train=True, "
                             "which adds the peer-visible bf16 token region")
        super().__init__(shape, device=group.device, rank=rank, world=group.world, padding=padding,
                         swiglu_limit=swiglu_limit, precision=precision)
        self.group, lay = group, group.layout
        ptrs = group.ptrs_for(rank)
        dev, L, H, k, W = self.device, shape.tokens, shape.hidden, shape.topk, group.world
        table = lambda off: torch.tensor([p + off for p in ptrs], dtype=torch.int64, device=dev)
        me_ptr = ptrs[rank]
        self.flags_peers, self.xq_peers, self.xsc_peers = table(lay.flags), table(lay.xq), table(lay.xsc)
        self.routes_peers, self.combine_peers = table(lay.routes_all), table(lay.combine)
        self.xsc_rows_peers = table(lay.xsc_rows)
        self.xsc_rows = tensor_from_ptr(ptrs[rank] + lay.xsc_rows, (L, H // 128), torch.int32, dev)
        self.pull_variant = "bulk"
        # combine push (and, in training, the input-gradient push) into receive streams: sequential
        # writes at the home rank instead of rows scattered to [token * topk + slot]
        self.stream_push = bool(lay.stream)
        if self.stream_push:
            self.recv_peers, self.recv_index_peers = table(lay.recv), table(lay.recv_index)
            self.recv = tensor_from_ptr(me_ptr + lay.recv, (W * L * k, H), torch.bfloat16, dev)
            self.recv_index = tensor_from_ptr(me_ptr + lay.recv_index, (L * k,), torch.int32, dev)
            self.stream_row = torch.empty(self.capacity, dtype=torch.int32, device=dev)
            # the schedule launches write the stream positions themselves when no counting chunk spans
            # two source ranks; otherwise a separate pass (plb_ep_stream_rows) follows the schedule
            self.schedule_writes_streams = (L * k) % 1024 == 0
            if self.schedule_writes_streams:
                nbytes = _lib.load().plb_moe_schedule_streams_scratch_bytes(W, L, k, self.num_local_experts)
                self.stream_scratch = torch.empty(max(nbytes, 4) // 4, dtype=torch.int32, device=dev)
        self._streamed = False
        self.linked, self.one_launch, self.one_launch_full = None, False, False   # attach_linked()
        me = ptrs[rank]
        self.xq = tensor_from_ptr(me + lay.xq, (L, H), torch.uint8, dev)
        self.xsc = tensor_from_ptr(me + lay.xsc, (L // 128, H // 128, 32, 16), torch.uint8, dev)
        self.routes_all = tensor_from_ptr(me + lay.routes_all, (W, L, k), torch.int32, dev)
        self.buffers["combine_buffer"] = tensor_from_ptr(me + lay.combine, (L * k, H), torch.bfloat16, dev)
        self.routes_local = torch.empty((L, k), dtype=torch.int32, device=dev)
        self.barrier_state = barrier_state_for(me + lay.flags, rank, dev)
        # Pushing GEMMs start `rank` source-rank blocks into their tile list: a block is the rows one
        # rank sends to one expert, L * k / E on average, in 256-row tiles.
        self.push_rotation = rank * max(1, (L * k // shape.experts) // 256) if W > 1 else 0
        # ... and step through the tiles a block and a bit at a time, so that the tiles in flight at
        # any moment belong to different home ranks
        self.push_stride = max(1, (L * k // shape.experts) // 256) + 1 if W > 1 else 1
        if lay.train:
            self.x_peers, self.d_out_peers = table(lay.x_bf16), table(lay.d_out)
            self.router_w_peers, self.d_x_rows_peers = table(lay.router_w), table(lay.d_x_rows)
            # the peer-visible copies replace the private buffers of the single-rank session
            self.x_buffer = tensor_from_ptr(me + lay.x_bf16, (L, H), torch.bfloat16, dev)
            self._x_storage = self.x_buffer     # tokens per rank is a multiple of 128: no padding rows
            self.router_weight_buffer = tensor_from_ptr(me + lay.router_w, (L, k), torch.float32, dev)
            self.d_out_buffer = tensor_from_ptr(me + lay.d_out, (L, H), torch.bfloat16, dev)
            self._d_x_rows = tensor_from_ptr(me + lay.d_x_rows, (L * k, H), torch.bfloat16, dev)
            if lay.stream:
                self.d_x_recv_peers = table(lay.d_x_recv)
                self.d_x_recv = tensor_from_ptr(me + lay.d_x_recv, (W * L * k, H), torch.bfloat16, dev)
            # The gate/up weight gradient needs the bf16 token rows of this rank's experts. They are the
            # same tokens the forward dispatched, so every peer's token buffer is copied whole early in
            # the backward, by the copy engines on a side stream (W * L rows: no more bytes than T * k
            # row pulls once top-k >= W, far fewer below), and the weight gradient gathers its rows locally.
            self.x_all = torch.empty((W, L, H), dtype=torch.bfloat16, device=dev)
            self.x_all_table = torch.tensor([self.x_all[q].data_ptr() for q in range(W)], dtype=torch.int64, device=dev)
            self._peer_x = [tensor_from_ptr(ptrs[q] + lay.x_bf16, (L, H), torch.bfloat16, dev) for q in range(W)]
            self.copy_stream = torch.cuda.Stream(dev)
            self._x_readable, self._x_gathered = torch.cuda.Event(), torch.cuda.Event()
            self._x_gather_pending = False

    def _alloc_train_buffers(self):
        super()._alloc_train_buffers()
        if self.group.layout.train:
            self.buffers["d_x_routed_buffer"] = self._d_x_rows

    # ---- steps, in the order forward() issues them
    def stage_inputs(self, inputs: mok.Inputs):
        self.x_buffer.copy_(inputs.x)
        self.router_weight_buffer.copy_(inputs.router)
        self.routes_local.copy_(inputs.experts)
        self.quantize_tokens()

    def publish_routes(self):
        _lib.call("plb_ep_publish", self.routes_local.data_ptr(), self.routes_local.numel() * 4,
                  self.routes_peers.data_ptr(), self.rank, self.world, mok._stream())

    def barrier(self):
        if self.group.distributed:
            _lib.call("plb_ep_barrier", self.flags_peers.data_ptr(), self.barrier_state.data_ptr(), self.rank,
                      self.world, self.status.buf.data_ptr(), mok._stream())

    def build_schedule(self):
        s, sh = self.schedule, self.shape
        if self.stream_push and self.schedule_writes_streams:
            _lib.call("plb_moe_schedule_streams", self.routes_all.data_ptr(), self.world, sh.tokens, sh.topk,
                      self.rank * self.num_local_experts, self.num_local_experts, self.capacity, self.padding,
                      s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(), s.dest_row.data_ptr(),
                      s.num_tokens.data_ptr(), s.tokens_per_expert.data_ptr(), s.expert_offsets.data_ptr(),
                      s.block_expert.data_ptr(), self.stream_scratch.data_ptr(), self.stream_scratch.numel() * 4,
                      self.rank, sh.tokens * sh.topk, self.stream_row.data_ptr(), self.recv_index_peers.data_ptr(),
                      self.status.buf.data_ptr(), mok._stream())
            return
        _lib.call("plb_moe_schedule", self.routes_all.data_ptr(), self.world, sh.tokens, sh.topk,
                  self.rank * self.num_local_experts, self.num_local_experts, self.capacity, self.padding,
                  s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(), s.dest_row.data_ptr(),
                  s.num_tokens.data_ptr(), s.tokens_per_expert.data_ptr(), s.expert_offsets.data_ptr(),
                  s.block_expert.data_ptr(), s.scratch.data_ptr(), s.scratch.numel() * 4,
                  self.status.buf.data_ptr(), mok._stream())

    def pull_bf16(self):
        """Dispatch of the bf16 routed precision: rows come from the home ranks' bf16 tokens."""
        s, b, sh = self.schedule, self.buffers, self.shape
        _lib.call("plb_ep_gather_rows", self.x_peers.data_ptr(), s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(),
                  s.num_tokens.data_ptr(), self.capacity, sh.hidden, b["x_routed_bf16"].data_ptr(), mok._stream())

    def stream_rows(self):
        """Positions of this rank's rows in the home ranks' receive streams, and the index the home
        ranks read their (token, slot) rows through."""
        s, sh = self.schedule, self.shape
        _lib.call("plb_ep_stream_rows", s.peer_rank.data_ptr(), s.dest_row.data_ptr(), s.num_tokens.data_ptr(),
                  self.capacity, self.rank, self.world, sh.tokens * sh.topk, self.stream_row.data_ptr(),
                  self.recv_index_peers.data_ptr(), mok._stream())

    def gemm_down_push(self, train: bool = False):
        s, b, w, sh = self.schedule, self.buffers, self.weights, self.shape
        self._streamed = self.stream_push and self.precision != "bf16"
        if self._streamed:
            if not self.schedule_writes_streams:
                self.stream_rows()
            _lib.call("plb_moe_gemm_down_push", b["hidden_routed_fp8"].data_ptr(), b["hidden_routed_sc"].data_ptr(),
                      w["w_routed_down_fp8"].data_ptr(), w["w_routed_down_sc"].data_ptr(),
                      s.block_expert.data_ptr(), s.num_tokens.data_ptr(), self.stream_row.data_ptr(),
                      s.peer_rank.data_ptr(), self.capacity, self.num_local_experts, sh.intermediate, sh.hidden,
                      self.push_rotation, self.push_stride, self.recv_peers.data_ptr(), self.status.buf.data_ptr(),
                      mok._stream())
            return
        if self.precision == "bf16":
            _lib.call("plb_moe_gemm_down_bf16", b["hidden_routed_bf16"].data_ptr(), w["w_routed_down_bf16"].data_ptr(),
                      s.block_expert.data_ptr(), s.num_tokens.data_ptr(), s.dest_row.data_ptr(), s.peer_rank.data_ptr(),
                      self.capacity, self.num_local_experts, sh.intermediate, sh.hidden, self.push_rotation, None,
                      self.combine_peers.data_ptr(), self.status.buf.data_ptr(), mok._stream())
            return
        _lib.call("plb_moe_gemm_down_push", b["hidden_routed_fp8"].data_ptr(), b["hidden_routed_sc"].data_ptr(),
                  w["w_routed_down_fp8"].data_ptr(), w["w_routed_down_sc"].data_ptr(),
                  s.block_expert.data_ptr(), s.num_tokens.data_ptr(), s.dest_row.data_ptr(),
                  s.peer_rank.data_ptr(), self.capacity, self.num_local_experts, sh.intermediate, sh.hidden,
                  self.push_rotation, self.push_stride, self.combine_peers.data_ptr(), self.status.buf.data_ptr(), mok._stream())

    def attach_linked(self, linked, full: bool = False):
        """Run the inference forward's expert FFN through the linked forward image (moe_linked.LinkedMoE on
        this host): dispatch warps, both projections and the combine push in ONE launch. With `full` the same
        launch also holds the group barrier and the weighted epilogue: everything after the schedule."""
        self.linked, self.one_launch, self.one_launch_full = linked, linked is not None, linked is not None and full

    def ffn_one_launch(self):
        """pull() + gemm_gate_up() + gemm_down_push() as one launch of the linked forward image; with the
        full image also barrier() + fwd_epilogue(), and the output is returned."""
        s = self.schedule
        self._streamed = self.stream_push
        if self._streamed and not self.schedule_writes_streams:
            self.stream_rows()
        if not self.fused_dispatch:
            self.pull()
        kw = dict(dispatch=self.fused_dispatch, dest_rows=self.stream_row if self._streamed else s.dest_row,
                  out_peers=self.recv_peers if self._streamed else self.combine_peers,
                  rotation=self.push_rotation, stride=self.push_stride)
        if not self.one_launch_full:
            self.linked.forward_ffn(**kw)
            return None
        if not self.group.distributed:
            raise ValueError("the full forward image waits for the other ranks inside the launch: real GPUs only")
        return self.linked.forward_full(combine=self.recv if self._streamed else self.buffers["combine_buffer"],
                                        index=self.recv_index if self._streamed else None, flags_peers=self.flags_peers,
                                        barrier_state=self.barrier_state, rank=self.rank, world=self.world, **kw)

    def fwd_epilogue(self, y_shared=None):
        if not self._streamed:
            return super().fwd_epilogue(y_shared)
        b, sh = self.buffers, self.shape
        _lib.call("plb_moe_fwd_epilogue_indexed", mok._ptr(y_shared), self.recv.data_ptr(), self.recv_index.data_ptr(),
                  self.router_weight_buffer.data_ptr(), sh.tokens, sh.topk, sh.hidden, b["output"].data_ptr(),
                  mok._stream())
        return b["output"]

    def start_token_gather(self):
        """Backward, once the d_y rows have been pulled: copy every rank's bf16 tokens here with the copy
        engines on the side stream, under the down-projection gradients and the SwiGLU backward (local
        work that leaves NVLink idle). Every rank's tokens have been in place since the forward's first
        barrier and stay until the backward's last one. (Issued in the forward, the copies shared the
        links with the dispatch: the pull took 1.14 ms instead of 0.44 on eight GPUs.)"""
        main = torch.cuda.current_stream()
        self._x_readable.record(main)
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self._x_readable)
            for q in range(self.world):
                self.x_all[q].copy_(self._peer_x[q], non_blocking=True)
            self._x_gathered.record(self.copy_stream)
        self._x_gather_pending = True

    def join_token_gather(self):
        """The copies have landed before anything queued after this call runs: called where the
        backward reads them, which is before its last barrier, so no rank can be overwriting its
        tokens for the next step while a peer still copies them."""
        if self._x_gather_pending:
            torch.cuda.current_stream().wait_event(self._x_gathered)
            self._x_gather_pending = False

    def device_step(self, train: bool = False):
        """Everything after the inputs sit in x_buffer / routes_local / router_weight_buffer."""
        self.quantize_tokens()
        self.publish_routes()
        self.barrier()          # routes gathered, every rank's quantised tokens readable
        self.build_schedule()
        if self.one_launch and not train:
            out = self.ffn_one_launch()
            if out is not None:
                return out          # the launch held the barrier and the epilogue too
        else:
            self.pull()
            if train:
                self.gemm_gate_up_train()
            else:
                self.gemm_gate_up()
            self.gemm_down_push(train)
        self.barrier()          # every rank's rows have landed in my combine buffer
        return self.fwd_epilogue()

    def forward_phases(self, train: bool = False):
        """device_step() as (name, call) pairs, for per-phase timing."""
        gate_up = self.gemm_gate_up_train if train else self.gemm_gate_up
        return [("quantise tokens", self.quantize_tokens), ("publish routes", self.publish_routes),
                ("barrier", self.barrier), ("schedule", self.build_schedule), ("dispatch pull", self.pull),
                ("gate/up GEMM", gate_up), ("down GEMM + push", lambda: self.gemm_down_push(train)),
                ("barrier ", self.barrier), ("epilogue", self.fwd_epilogue)]

    def backward_phases(self):
        """backward() as (name, call) pairs (d_out already staged in d_out_buffer)."""
        return [("bwd barrier", self.barrier), ("router gradient", self.bwd_home_side_early),
                ("d_y pull", self.bwd_pull_dy), ("token copies (side stream)", self.bwd_start_token_gather),
                ("down dgrad + wgrad", self.bwd_down),
                ("SwiGLU backward", self.bwd_activation), ("gate/up dgrad + d_x push", self.bwd_push_dx),
                ("x pull + gate/up wgrad", self.bwd_gate_up_wgrad), ("bwd barrier ", self.barrier),
                ("slot sum", self.bwd_home_side_late)]

    def forward(self, inputs: mok.Inputs, *, check: bool = True, train: bool = False):
        if not self.group.distributed:
            raise ValueError("ranks of a LocalGroup are stepped together: use forward_local_group()")
        self.status.reset()
        self.x_buffer.copy_(inputs.x)
        self.router_weight_buffer.copy_(inputs.router)
        self.routes_local.copy_(inputs.experts)
        out = self.device_step(train)
        if check:
            self.status.check("after EP forward")
        return {"output": out, **self.context_tensors()}

    # ---- backward, in the order backward() issues the steps (mirror of dispatch / combine)
    def bwd_pull_dy(self):
        """d_y rows of this rank's experts: w * d_out pulled from the tokens' home ranks."""
        s, b, sh = self.schedule, self.buffers, self.shape
        _lib.call("plb_ep_bwd_dy", self.d_out_peers.data_ptr(), self.router_w_peers.data_ptr(), s.peer_rank.data_ptr(),
                  s.peer_token_idx.data_ptr(), s.dest_row.data_ptr(), s.num_tokens.data_ptr(), self.capacity, sh.hidden,
                  b["d_y_routed"].data_ptr(), mok._stream())

    def bwd_down(self):
        """Down projection: data gradient d_hidden, then the weight gradient over each expert's rows."""
        b, w, sh = self.buffers, self.weights, self.shape
        H, I = sh.hidden, sh.intermediate
        if self.precision == "bf16":
            self._rows_gemm_bf16(b["d_y_routed"], w["w_down_t_bf16"], H, I, b["d_hidden_routed"], self._identity_rows)
            self._wgrad_bf16(b["d_y_routed"], b["t_rows_h"], b["hidden_routed_bf16"], b["t_rows_i"], b["d_w_routed_down"])
            return
        dy_q, dy_sc, dy_t, dy_t_sc = mok.mxfp8_quantize(b["d_y_routed"], True, True, self.schedule.num_tokens)
        self._gemm_rows(dy_q, dy_sc, w["w_down_t_fp8"], w["w_down_t_sc"], H, I, b["d_hidden_routed"], self._identity_rows)
        _, _, h_t, h_t_sc = mok.mxfp8_quantize(b["hidden_routed_bf16"], False, True, self.schedule.num_tokens)
        self._wgrad(dy_t, dy_t_sc, h_t, h_t_sc, H, I, b["d_w_routed_down"])

    def bwd_activation(self):
        s, b, sh = self.schedule, self.buffers, self.shape
        self.select_activation()
        if self.precision == "bf16":
            _lib.call("plb_moe_swiglu_bwd_bf16", b["gate_routed_bf16"].data_ptr(), b["up_routed_bf16"].data_ptr(),
                      b["d_hidden_routed"].data_ptr(), s.num_tokens.data_ptr(), self.capacity, sh.intermediate,
                      b["d_gate_up_routed"].data_ptr(), mok._stream())
            return
        _lib.call("plb_moe_swiglu_bwd", b["gate_routed_fp8"].data_ptr(), b["gate_routed_sc"].data_ptr(),
                  b["up_routed_fp8"].data_ptr(), b["up_routed_sc"].data_ptr(), b["d_hidden_routed"].data_ptr(),
                  s.num_tokens.data_ptr(), self.capacity, sh.intermediate, b["d_gate_up_routed"].data_ptr(), mok._stream())
        self._dgu = mok.mxfp8_quantize(b["d_gate_up_routed"], True, True, self.schedule.num_tokens)

    def bwd_push_dx(self):
        """Gate/up data gradient: d_x rows leave the GEMM epilogue straight into the home rank's
        [tokens * topk, H] buffer."""
        s, w, sh = self.schedule, self.weights, self.shape
        if self.precision == "bf16":
            # the bf16 GEMM's epilogue pushes to [token * topk + slot] of the home rank (no receive streams)
            _lib.call("plb_moe_gemm_down_bf16", self.buffers["d_gate_up_routed"].data_ptr(), w["w_cat_t_bf16"].data_ptr(),
                      s.block_expert.data_ptr(), s.num_tokens.data_ptr(), s.dest_row.data_ptr(), s.peer_rank.data_ptr(),
                      self.capacity, self.num_local_experts, 2 * sh.intermediate, sh.hidden, self.push_rotation, None,
                      self.d_x_rows_peers.data_ptr(), self.status.buf.data_ptr(), mok._stream())
            return
        dgu_q, dgu_sc, _, _ = self._dgu
        # with receive streams the rows take the positions the forward's combine rows took (same schedule)
        dest, peers = (self.stream_row, self.d_x_recv_peers) if self._streamed else (s.dest_row, self.d_x_rows_peers)
        _lib.call("plb_moe_gemm_down_push", dgu_q.data_ptr(), dgu_sc.data_ptr(), w["w_cat_t_fp8"].data_ptr(),
                  w["w_cat_t_sc"].data_ptr(), s.block_expert.data_ptr(), s.num_tokens.data_ptr(), dest.data_ptr(),
                  s.peer_rank.data_ptr(), self.capacity, self.num_local_experts, 2 * sh.intermediate, sh.hidden,
                  self.push_rotation, self.push_stride, peers.data_ptr(), self.status.buf.data_ptr(), mok._stream())

    def bwd_gate_up_wgrad(self):
        """Gate/up weight gradient: the bf16 token rows pulled from their home ranks, quantised along the rows."""
        s, b, sh = self.schedule, self.buffers, self.shape
        if self.precision == "bf16":
            # the bf16 rows the forward's dispatch gathered are still in place
            self._wgrad_bf16(b["d_gate_up_routed"], b["t_rows_2i"], b["x_routed_bf16"], b["t_rows_h2"], b["d_w_routed_gate_up"])
            return
        _, _, dgu_t, dgu_t_sc = self._dgu
        # rows come from the copies the forward made of every rank's tokens (local reads); without a
        # training forward in front (a LocalGroup stepping phases by hand) they are pulled from the peers
        src = self.x_peers
        if self._x_gather_pending:
            self.join_token_gather()
            src = self.x_all_table
        _lib.call("plb_ep_gather_rows", src.data_ptr(), s.peer_rank.data_ptr(), s.peer_token_idx.data_ptr(),
                  s.num_tokens.data_ptr(), self.capacity, sh.hidden, b["x_routed_bf16"].data_ptr(), mok._stream())
        _, _, x_t, x_t_sc = mok.mxfp8_quantize(b["x_routed_bf16"], False, True, self.schedule.num_tokens)
        self._wgrad(dgu_t, dgu_t_sc, x_t, x_t_sc, 2 * sh.intermediate, sh.hidden, b["d_w_routed_gate_up"])
        self._dgu = None

    def bwd_start_token_gather(self):
        if self.group.layout.train and self.group.distributed and self.precision == "mxfp8":
            self.start_token_gather()

    def bwd_expert_side(self):
        """Everything this rank does for the rows of ITS experts: pull w * d_out from the tokens'
        home ranks, both data gradients, SwiGLU backward, the three weight gradients, and the push
        of the input-gradient rows back to the home ranks."""
        self.bwd_pull_dy()
        self.bwd_start_token_gather()
        self.bwd_down()
        self.bwd_activation()
        self.bwd_push_dx()
        self.bwd_gate_up_wgrad()

    def bwd_home_side_early(self):
        """Needs only this rank's own tokens: the router-weight gradient."""
        b, sh = self.buffers, self.shape
        if self._streamed:
            _lib.call("plb_moe_router_grad_indexed", self.d_out_buffer.data_ptr(), self.recv.data_ptr(),
                      self.recv_index.data_ptr(), sh.tokens, sh.topk, sh.hidden, b["d_router_weights"].data_ptr(),
                      mok._stream())
            return
        _lib.call("plb_moe_router_grad", self.d_out_buffer.data_ptr(), b["combine_buffer"].data_ptr(), sh.tokens, sh.topk,
                  sh.hidden, b["d_router_weights"].data_ptr(), mok._stream())

    def bwd_home_side_late(self):
        """After every rank's input-gradient rows have landed: sum the slots of each token."""
        b, sh = self.buffers, self.shape
        if self._streamed:
            _lib.call("plb_moe_fwd_epilogue_indexed", None, self.d_x_recv.data_ptr(), self.recv_index.data_ptr(),
                      self._ones.data_ptr(), sh.tokens, sh.topk, sh.hidden, b["d_x"].data_ptr(), mok._stream())
            return
        _lib.call("plb_moe_fwd_epilogue", None, b["d_x_routed_buffer"].data_ptr(), self._ones.data_ptr(), sh.tokens,
                  sh.topk, sh.hidden, b["d_x"].data_ptr(), mok._stream())

    def gradients(self):
        b, I = self.buffers, self.shape.intermediate
        g = b["d_w_routed_gate_up"]
        return {"d_x": b["d_x"], "d_router_weights": b["d_router_weights"], "d_w_routed_gate": g[:, :I],
                "d_w_routed_up": g[:, I:], "d_w_routed_down": b["d_w_routed_down"]}

    def backward(self, d_out: torch.Tensor, *, check: bool = True):
        """Backward of the last ``forward(train=True)`` of a distributed group."""
        if not self.group.distributed:
            raise ValueError("ranks of a LocalGroup are stepped together: use backward_local_group()")
        self.d_out_buffer.copy_(d_out)
        self.barrier()          # every rank's d_out is readable; forward's combine rows are long in place
        self.bwd_home_side_early()
        self.bwd_expert_side()
        self.barrier()          # every rank's d_x rows have landed here
        self.bwd_home_side_late()
        if check:
            self.status.check("after EP backward")
        return self.gradients()


def backward_local_group(hosts, d_out_per_rank):
    """Backward of forward_local_group(..., train=True), phase by phase on the current stream."""
    for h, d in zip(hosts, d_out_per_rank):
        h.d_out_buffer.copy_(d)
    for h in hosts:
        h.bwd_home_side_early()
        h.bwd_expert_side()
    for h in hosts:
        h.bwd_home_side_late()
        h.status.check("after local-group backward")
    return [h.gradients() for h in hosts]


def forward_local_group(hosts, inputs_per_rank, train: bool = False):
    """Run every rank of a LocalGroup phase by phase on the current stream."""
    for h, inp in zip(hosts, inputs_per_rank):
        h.status.reset()
        h.stage_inputs(inp)
        h.publish_routes()
    for h in hosts:
        h.build_schedule()
        h.pull()
        if train:
            h.gemm_gate_up_train()
        else:
            h.gemm_gate_up()
    for h in hosts:
        h.gemm_down_push(train)
    outs = [h.fwd_epilogue() for h in hosts]
    for h in hosts:
        h.status.check("after local-group forward")
    return outs


STREAM_PUSH_MIN_WORLD = 4


class BenchSession:
    """One rank of an IpcGroup with synthetic weights and inputs, stepped by the benchmark: the
    expert-parallel workload at 8192 tokens per rank, forward or forward + backward."""

    launches_per_step = 12  # quantise, scale rows, publish, barrier x2, schedule x3, pull, 2 GEMMs, epilogue
    # backward adds: barrier x2, router grad, d_y pull, 5 quantise, 2 dgrad GEMMs, SwiGLU backward, x gather,
    # 2 wgrad GEMMs, slot sum, 2 tail-zeroing launches
    launches_per_step_train = 12 + 18

    def __init__(self, shape: mok.Shape, dev, rank: int, world: int, train: bool = False, fused_dispatch: bool = False):
        self.shape, self.dev, self.train = shape, dev, train
        # receive streams pay once the combine rows scatter over several peers: no gain at two ranks,
        # 0.55 ms faster per push at eight
        self.group = IpcGroup(shape, rank, world, dev, train=train, stream=world >= STREAM_PUSH_MIN_WORLD)
        self.host = EpMoKHost(shape, rank, self.group)
        self.host.fused_dispatch = fused_dispatch
        if self.host.stream_push and not self.host.schedule_writes_streams:
            self.launches_per_step = self.launches_per_step + 1     # the separate stream-position pass
        torch.manual_seed(1234 + rank)
        E, H, I = self.host.num_local_experts, shape.hidden, shape.intermediate
        if train:
            mk = lambda *sh: (torch.randn(*sh, device=dev) * 0.02).to(torch.bfloat16)
            self.host.load_weights(mk(E, I, H), mk(E, I, H), mk(E, H, I), keep_unpacked=False, train=True)
            self.d_out = torch.randn(shape.tokens, H, device=dev).to(torch.bfloat16)
            self.launches_per_step = self.launches_per_step_train
        else:
            q = {}
            for name, rows, cols in (("gate", I, H), ("up", I, H), ("down", H, I)):
                fp8 = torch.empty((E, rows, cols), dtype=torch.uint8, device=dev)
                sc = torch.empty((E * rows // 128, cols // 128, 32, 16), dtype=torch.uint8, device=dev)
                for e in range(E):
                    w = (torch.randn(rows, cols, device=dev) * 0.02).to(torch.bfloat16)
                    a, b, _, _ = mok.mxfp8_quantize(w)
                    fp8[e].copy_(a)
                    sc[e * rows // 128:(e + 1) * rows // 128].copy_(b)
                q[name] = (fp8, sc)
            self.host.load_quantized_weights(*q["gate"], *q["up"], *q["down"], keep_unpacked=False)
        logits = torch.randn(shape.tokens, shape.experts, device=dev)
        values, experts = torch.topk(logits, shape.topk, dim=1)
        x = torch.randn(shape.tokens, H, device=dev).to(torch.bfloat16)
        self.inputs = mok.Inputs(x, experts, torch.softmax(values.float(), dim=-1))
        h = self.host
        h.x_buffer.copy_(x)
        h.router_weight_buffer.copy_(self.inputs.router)
        h.routes_local.copy_(experts)
        self.kernel_events = []
        self.h_x = x.cpu().pin_memory()
        self.h_routes = experts.to(torch.int32).cpu().pin_memory()
        self.h_router = self.inputs.router.cpu().pin_memory()
        self.h_out = torch.empty((shape.tokens, H), dtype=torch.bfloat16).pin_memory()
        torch.cuda.synchronize()

    def step(self, record=False):
        h = self.host
        h.quantize_tokens()
        h.publish_routes()
        h.barrier()
        h.build_schedule()
        if h.one_launch and not self.train:
            if h.ffn_one_launch() is None:
                h.barrier()
                h.fwd_epilogue()
            return
        h.pull()
        gate_up = h.gemm_gate_up_train if self.train else h.gemm_gate_up
        if record:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            gate_up()
            b.record()
            self.kernel_events.append((a, b))
        else:
            gate_up()
        h.gemm_down_push(self.train)
        h.barrier()
        h.fwd_epilogue()
        if self.train:
            h.backward(self.d_out, check=False)

    def check(self):
        self.host.status.check("bench (EP)")

    def choose_dispatch(self, steps: int = 6):
        """Decide the form of the expert FFN by timing it: `steps` steps with the pull kernel in front of
        the gate/up GEMM, `steps` with the dispatch warps inside it and, when the linked images are
        there, `steps` with the whole FFN (dispatch warps, both projections, combine push) as ONE
        launch of the linked forward image; device time, slowest rank; the fastest stays on. Whether
        rows arriving under the mainloop beat rows fetched before it depends on how many of them are
        remote, so it is measured on the group at hand. Returns the times in ms per step. Forward
        sessions of the MXFP8 precision only."""
        import torch.distributed as dist
        h = self.host
        if self.train or h.precision != "mxfp8" or h.shape.hidden > 4096:
            return None
        times, failed = {}, None
        forms = [("pull kernel", False, False), ("in-kernel", True, False)]
        linked = None
        try:
            from . import moe_linked
            linked = moe_linked.LinkedMoE(h)
            forms.append(("one launch (linked image)", True, True))
            forms.append(("whole forward in one launch (linked image)", True, "full"))
        except Exception:  # noqa: BLE001 - images absent: the library's launches are timed alone
            linked = None
        for name, fused, one in forms:
            h.fused_dispatch = fused
            h.attach_linked(linked if one else None, full=one == "full")
            for _ in range(2):
                self.step()
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                self.step()
            b.record()
            torch.cuda.synchronize()
            # a form that reports a device status on any rank is out, whatever its time
            bad = torch.tensor([int(h.status.buf[0].item() != 0)], dtype=torch.int32, device=self.dev)
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
            if bad.item():
                failed = name if failed is None else f"{failed}, {name}"
                h.status.reset()
                torch.cuda.synchronize()
                dist.barrier()
                continue
            t = torch.tensor([a.elapsed_time(b) / steps], dtype=torch.float64, device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times[name] = float(t.item())
        if "pull kernel" not in times:
            raise RuntimeError("the expert-parallel step reports a device status with the pull kernel")
        chosen = min(times, key=times.get)
        _, fused, one = next(f for f in forms if f[0] == chosen)
        h.fused_dispatch = fused
        h.attach_linked(linked if one else None, full=one == "full")
        if linked is not None and not one:
            linked.close()
        out = {"ms_per_step": times, "chosen": chosen}
        if failed:
            out["rejected"] = f"{failed}: device status during its timing"
        return out

    def traffic_per_launch(self):
        return None

    def e2e(self, steps):
        """Pinned host buffers in and out every step through EpHostPipeline; device-timed from the
        first submit to the last result leaving the device."""
        pipe = EpHostPipeline(self.host)
        outs = [self.h_out, torch.empty_like(self.h_out).pin_memory()]
        for i in range(2):
            pipe.submit(self.h_x, self.h_routes, self.h_router, outs[i % 2])
        pipe.drain()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(steps):
            pipe.submit(self.h_x, self.h_routes, self.h_router, outs[i % 2])
        b.record(pipe.copy_out)
        pipe.drain()
        self.host.status.check("bench (EP e2e)")
        h2d = self.h_x.numel() * 2 + self.h_routes.numel() * 4 + self.h_router.numel() * 4
        return a.elapsed_time(b) / steps, h2d, self.h_out.numel() * 2


class EpHostPipeline:
    """mok.HostPipeline for one rank of a distributed group: inputs of step i+1 travel host -> device
    and the result of step i-1 device -> host on side streams while step i (with its group barriers)
    runs on the current stream. Every rank must submit the same number of steps."""

    def __init__(self, host: EpMoKHost):
        self.host, dev = host, host.device
        L, H, k = host.shape.tokens, host.shape.hidden, host.shape.topk
        self.copy_in, self.copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.x = [torch.empty((L, H), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        self.routes = [torch.empty((L, k), dtype=torch.int32, device=dev) for _ in range(2)]
        self.router = [torch.empty((L, k), dtype=torch.float32, device=dev) for _ in range(2)]
        self.out = [torch.empty((L, H), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        ev = lambda: [torch.cuda.Event() for _ in range(2)]
        self.in_ready, self.in_free, self.out_ready, self.out_free = ev(), ev(), ev(), ev()
        self.step = 0

    def submit(self, h_x, h_routes, h_router, h_out):
        host, i = self.host, self.step % 2
        compute = torch.cuda.current_stream()
        with torch.cuda.stream(self.copy_in):
            if self.step >= 2:
                self.copy_in.wait_event(self.in_free[i])
            self.x[i].copy_(h_x, non_blocking=True)
            self.routes[i].copy_(h_routes, non_blocking=True)
            self.router[i].copy_(h_router, non_blocking=True)
            self.in_ready[i].record(self.copy_in)
        compute.wait_event(self.in_ready[i])
        host.x_buffer.copy_(self.x[i])
        host.routes_local.copy_(self.routes[i])
        host.router_weight_buffer.copy_(self.router[i])
        self.in_free[i].record(compute)
        result = host.device_step()
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
