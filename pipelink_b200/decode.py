"""Host side of the batch-1 decode interpreter: model tensors, the per-SM instruction schedule,
the argument block of ``plb_decode_step`` and a greedy decode loop.

Counterpart of the reference's decode host (campaigns/megakernel/host/export_inputs.py builds
the seeded model, KV caches and the ``instructions (1, num_sms, n, 32)`` tensor;
campaigns/megakernel/host/mk_host_abi.h:47-85 is the argument block). The schedule here gives
every SM one contiguous slice of each matvec's rows per layer (so a token costs about six
instructions per layer per SM), spreads the 8 x P partial-attention tasks over the SMs, and
orders work through one counter per (layer, opcode).
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib
from .mok import DeviceStatus, _stream

HIDDEN, Q_HEADS, KV_HEADS, HEAD_DIM, FFN = 2048, 32, 8, 64, 8192
QKV_ROWS = (Q_HEADS + 2 * KV_HEADS) * HEAD_DIM
OP_QKV, OP_ATTN, OP_REDUCE, OP_OPROJ, OP_UPGATE, OP_DOWN, OP_LMHEAD, OP_SAMPLE = 1, 2, 3, 4, 5, 6, 7, 8


class DecodeArgs(ctypes.Structure):
    """plb_decode_args (include/pipelink_b200.h), same field order."""
    _fields_ = ([(n, ctypes.c_void_p) for n in (
        "qkv_w", "o_w", "up_w", "gate_w", "down_w", "attn_norm", "mlp_norm", "lm_norm", "lm_head",
        "k_cache", "v_cache", "rope_cos", "rope_sin", "hidden", "q_post_rope", "attn_out", "silu_out",
        "logits", "attn_out_partial", "attn_lse_partial", "argmax_val", "argmax_idx", "bars",
        "instructions", "pos_dev", "token_out", "status")] +
        [(n, ctypes.c_int32) for n in ("num_instructions", "max_seq_len", "max_parts", "vocab")] +
        [("attn_scale", ctypes.c_float), ("eps", ctypes.c_float), ("num_bars", ctypes.c_int32),
         ("layers", ctypes.c_int32)])


def split_even(units: int, parts: int):
    """units split into at most `parts` contiguous non-empty (start, count) slices, sizes within 1."""
    parts = min(parts, units)
    base, extra = divmod(units, parts)
    out, start = [], 0
    for i in range(parts):
        n = base + (1 if i < extra else 0)
        out.append((start, n))
        start += n
    return out


def build_schedule(num_sms: int, layers: int, vocab: int, partitions: int, fuse_reduce: bool = True):
    """Returns (instructions i32 [num_sms, n, 32] as a CPU tensor, number of counters).

    With `fuse_reduce` the partitions of a KV head count themselves in on one extra counter per
    (layer, KV head) and the last to arrive merges the head's partials, so opcode 3 is not
    emitted and a layer has five dependent stages instead of six."""
    if vocab // 2 < num_sms:
        raise ValueError("vocab too small: every SM must own an LM-head slice")
    per_sm = [[] for _ in range(num_sms)]
    bar = lambda layer, op: layer * 8 + op
    rr = 0  # rotating start so small ops do not always land on SM 0

    def emit(sm, op, layer, a0, a1, a2, dep, target, sig, a3=0):
        per_sm[sm].append([op, layer, a0, a1, a2, a3, dep, target, sig] + [0] * 23)

    arrive = lambda layer, kvh: (layers + 1) * 8 + layer * KV_HEADS + kvh

    n_down_prev = 0
    for l in range(layers):
        dep, target = (-1, 0) if l == 0 else (bar(l - 1, OP_DOWN), n_down_prev)
        qkv = split_even(QKV_ROWS // 2, num_sms)
        for sm, (s, n) in enumerate(qkv):
            emit(sm, OP_QKV, l, 2 * s, 2 * n, 0, dep, target, bar(l, OP_QKV))
        for t in range(KV_HEADS * partitions):
            if fuse_reduce:
                emit((rr + t) % num_sms, OP_ATTN, l, t // partitions, partitions, t % partitions,
                     bar(l, OP_QKV), len(qkv), bar(l, OP_REDUCE), 1 + arrive(l, t // partitions))
            else:
                emit((rr + t) % num_sms, OP_ATTN, l, t // partitions, partitions, t % partitions,
                     bar(l, OP_QKV), len(qkv), bar(l, OP_ATTN))
        rr = (rr + KV_HEADS * partitions) % num_sms
        if not fuse_reduce:
            for kvh in range(KV_HEADS):
                emit((rr + kvh) % num_sms, OP_REDUCE, l, kvh * 4, 4, partitions, bar(l, OP_ATTN),
                     KV_HEADS * partitions, bar(l, OP_REDUCE))
            rr = (rr + KV_HEADS) % num_sms
        oproj = split_even(HIDDEN // 2, num_sms)
        for sm, (s, n) in enumerate(oproj):
            emit(sm, OP_OPROJ, l, 2 * s, 2 * n, 0, bar(l, OP_REDUCE), KV_HEADS, bar(l, OP_OPROJ))
        upgate = split_even(FFN, num_sms)
        for sm, (s, n) in enumerate(upgate):
            emit(sm, OP_UPGATE, l, s, n, 0, bar(l, OP_OPROJ), len(oproj), bar(l, OP_UPGATE))
        down = split_even(HIDDEN // 2, num_sms)
        for sm, (s, n) in enumerate(down):
            emit(sm, OP_DOWN, l, 2 * s, 2 * n, 0, bar(l, OP_UPGATE), len(upgate), bar(l, OP_DOWN))
        n_down_prev = len(down)
    lm = split_even(vocab // 2, num_sms)
    for sm, (s, n) in enumerate(lm):
        emit(sm, OP_LMHEAD, 0, 2 * s, 2 * n, 0, bar(layers - 1, OP_DOWN), n_down_prev, bar(layers, OP_LMHEAD))
    emit(0, OP_SAMPLE, 0, len(lm), 0, 0, bar(layers, OP_LMHEAD), len(lm), -1)
    n = max(len(x) for x in per_sm)
    inst = torch.zeros((num_sms, n, 32), dtype=torch.int32)
    for sm, rows in enumerate(per_sm):
        if rows:
            inst[sm, : len(rows)] = torch.tensor(rows, dtype=torch.int32)
    return inst, (layers + 1) * 8 + layers * KV_HEADS


def rope_tables(rows: int, theta=500000.0, factor=32.0, low=1.0, high=4.0, original=8192):
    """llama3-scaled RoPE tables, f32 [rows, 32] (config: export_inputs.py:104-112)."""
    i = torch.arange(HEAD_DIM // 2, dtype=torch.float64)
    inv = 1.0 / theta ** (2.0 * i / HEAD_DIM)
    wavelen = 2.0 * math.pi / inv
    smooth = (original / wavelen - low) / (high - low)
    scaled = torch.where(wavelen > original / low, inv / factor,
                         torch.where(wavelen < original / high, inv, (1 - smooth) * inv / factor + smooth * inv))
    ang = torch.arange(rows, dtype=torch.float64)[:, None] * scaled[None, :]
    return torch.cos(ang).float(), torch.sin(ang).float()


class DecodeSession:
    """Weights, caches, activations and the instruction stream for one model on one GPU."""

    def __init__(self, weights: dict, *, max_seq_len: int, device="cuda", partitions: int | None = None,
                 num_sms: int | None = None, fuse_reduce: bool = True):
        _lib.load()
        self.device = torch.device(device)
        dev = self.device
        self.w = {k: v.to(device=dev, dtype=torch.bfloat16).contiguous() for k, v in weights.items()}
        self.layers = self.w["qkv_w"].shape[0]
        self.vocab = self.w["lm_head"].shape[0]
        self.max_seq_len = max_seq_len
        self.num_sms = num_sms or torch.cuda.get_device_properties(dev).multi_processor_count
        self.partitions = partitions or max(1, self.num_sms // KV_HEADS)
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.k_cache = torch.zeros((self.layers, max_seq_len, KV_HEADS, HEAD_DIM), **bf)
        self.v_cache = torch.zeros_like(self.k_cache)
        cos, sin = rope_tables(max_seq_len)
        self.rope_cos, self.rope_sin = cos.to(dev).contiguous(), sin.to(dev).contiguous()
        self.hidden = torch.zeros(HIDDEN, **bf)
        self.q_post_rope = torch.zeros(HIDDEN, **bf)
        self.attn_out = torch.zeros(HIDDEN, **bf)
        self.silu_out = torch.zeros(FFN, **bf)
        self.logits = torch.zeros(self.vocab, **bf)
        self.attn_out_partial = torch.zeros((Q_HEADS, self.partitions, HEAD_DIM), dtype=torch.float32, device=dev)
        self.attn_lse_partial = torch.zeros((Q_HEADS, self.partitions), dtype=torch.float32, device=dev)
        self.argmax_val = torch.zeros(self.num_sms, dtype=torch.float32, device=dev)
        self.argmax_idx = torch.zeros(self.num_sms, dtype=torch.int32, device=dev)
        inst, nbars = build_schedule(self.num_sms, self.layers, self.vocab, self.partitions, fuse_reduce)
        self.instructions = inst.to(dev).contiguous()
        self.bars = torch.zeros(nbars, dtype=torch.int32, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self.token_out = torch.full((max_seq_len + 1,), -1, dtype=torch.int32, device=dev)
        self.status = DeviceStatus(dev)
        a = DecodeArgs()
        for name in ("qkv_w", "o_w", "up_w", "gate_w", "down_w", "attn_norm", "mlp_norm", "lm_norm", "lm_head"):
            setattr(a, name, self.w[name].data_ptr())
        for name in ("k_cache", "v_cache", "rope_cos", "rope_sin", "hidden", "q_post_rope", "attn_out", "silu_out",
                     "logits", "attn_out_partial", "attn_lse_partial", "argmax_val", "argmax_idx", "bars",
                     "instructions", "token_out"):
            setattr(a, name, getattr(self, name).data_ptr())
        a.pos_dev, a.status = self.pos.data_ptr(), self.status.buf.data_ptr()
        a.num_instructions, a.max_seq_len = self.instructions.shape[1], max_seq_len
        a.max_parts, a.vocab = self.partitions, self.vocab
        a.attn_scale, a.eps, a.num_bars, a.layers = 1.0 / math.sqrt(HEAD_DIM), 1e-5, nbars, self.layers
        self.args = a

    def start(self, token_id: int, pos: int):
        """Place the embedding of `token_id` in the residual stream; it will be decoded at `pos`."""
        self.hidden.copy_(self.w["lm_head"][token_id])
        self.pos.fill_(pos)
        self.status.reset()

    def step(self):
        """Decode one token: one cooperative launch; the kernel itself advances pos and hidden."""
        _lib.call("plb_decode_step", ctypes.byref(self.args), self.num_sms, _stream())

    def decode(self, steps: int, check: bool = True):
        for _ in range(steps):
            self.step()
        if check:
            self.status.check("after decode")
        return self.token_out

    def bytes_per_token(self, pos: int) -> int:
        """Algorithmic HBM bytes of one token: every weight once + the KV rows read."""
        per_layer = (QKV_ROWS * HIDDEN + HIDDEN * HIDDEN + 2 * FFN * HIDDEN + HIDDEN * FFN) * 2
        kv = 2 * KV_HEADS * HEAD_DIM * 2 * (pos + 1)
        return self.layers * (per_layer + kv) + self.vocab * HIDDEN * 2
