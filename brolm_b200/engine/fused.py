"""Decode steps of few tokens as chains of operations in one persistent kernel.

A decode step of up to 16 tokens is a stream of weights; run part by part it
is a chain of some eight dependent kernels per layer, and what the boundaries
between them cost is of the order of the products themselves.  When every
block of a model is made of the parts this module knows (RMSNorm norms, the
Attention mixer with rotary positions, the gated feed-forward, bfloat16
weights), the step is compiled once per (model, cache) into lists of
operations for ``kernels.decode_chain``:

    [norm, qkv, rope]  attention(0)  [o, norm, gate_up, down, norm, qkv, rope]
    attention(1)  ...  attention(L-1)  [o, norm, gate_up, down, norm, head]

The attention over the cache stays the mixer's own kernel; everything between
two attentions is one launch whose weight stream does not stop.  The parts
keep their meaning: this is another way of running the same schedule, with
the same float32 residual stream, norm statistics and rotation, and a model
with any other part (or float32 weights) simply does not get a plan and runs
part by part.

The chains are off unless the environment has BROLM_CHAIN=1.  Measured on a
B200 at the sizes of Gemma 2 2B with 8 tokens, a layer's seven operations take
about 70 us inside the chain against about 60 us for the same work as separate
kernels with programmatic dependent launch: the products themselves stream at
the memory's full rate (155 MB in 19 us, the ring is refilled while the blocks
wait), but each of the seven barriers costs 2 us and a NORM operation, one
block per row, 6 to 10 us.  ``kernels.decode_chain(trace=...)`` gives the time
stamps these figures come from.

What the chain computes for a block (wlejon/brolm src/gemma2.cpp:345-387):
    x = pre_mixer(h); h += post_mixer(mixer(x)); x = pre_ffn(h); h += post_ffn(ffn(x))
"""
from __future__ import annotations

import os
import struct
from typing import Optional

import torch

from .. import kernels
from ..kernels import CHAIN_FIELDS as F
from ..parts.attention import Attention
from ..parts.block import Block
from ..parts.feedforward import GatedFeedForward
from ..parts.norm import RMSNorm
from ..parts.position import RotaryEmbedding

ROWS = kernels.CHAIN_MAX_TOKENS
MAX_SPLIT = 8
MAX_HIDDEN = 4608


def _bits(x: float) -> int:
    return struct.unpack("<q", struct.pack("<d", float(x)))[0]


def choose_split(row_tiles: int, k_blocks: int, sms: int, max_split: int = MAX_SPLIT) -> tuple[int, int]:
    """(slices of K, K blocks per slice) so that the busiest block streams the fewest tiles."""
    best = None
    for want in range(1, min(max_split, k_blocks) + 1):
        per = (k_blocks + want - 1) // want
        slices = (k_blocks + per - 1) // per
        rounds = (row_tiles * slices + sms - 1) // sms
        cost = (rounds * per, slices)
        if best is None or cost < best[0]:
            best = (cost, slices, per)
    return best[1], best[2]


def _norm_ok(n, dtype) -> bool:
    return n is None or (type(n) is RMSNorm and n.weight.dtype == dtype and n.weight.is_contiguous()
                         and n.weight.data_ptr() % 8 == 0)


def supported(model) -> Optional[str]:
    """None if the model's decode step can run as chains; otherwise the reason why not."""
    bf = torch.bfloat16
    if model.dtype != bf or model.device.type != "cuda":
        return "not a bfloat16 model on a GPU"
    if os.environ.get("BROLM_CHAIN") != "1":
        return "not asked for (BROLM_CHAIN=1 turns the chains on)"
    lay = model.layout
    H = lay.embedding.hidden
    if H % 8 or H > MAX_HIDDEN:
        return f"width {H}"
    if model.head.dtype != bf or model.head.stride(1) != 1 or model.head.stride(0) % 8 or model.head.data_ptr() % 16:
        return "output matrix"
    if type(model.final_norm) is not RMSNorm or not _norm_ok(model.final_norm, bf):
        return "final norm"
    for blk in model.blocks:
        if type(blk) is not Block or type(blk.mixer) is not Attention or type(blk.feedforward) is not GatedFeedForward:
            return "a block with other parts"
        for n in (blk.pre_mixer_norm, blk.pre_ffn_norm, blk.post_mixer_norm, blk.post_ffn_norm):
            if not _norm_ok(n, bf):
                return "a norm that is no bfloat16 RMSNorm"
            if n is not None and n.size != H:
                return "a norm of another width"
        if blk.pre_mixer_norm is None or blk.pre_ffn_norm is None:
            return "a block without pre-norms"
        a, f = blk.mixer, blk.feedforward
        if a.w_qkv.dtype != bf or a.w_o.dtype != bf or f.w_gate_up.dtype != bf or f.w_down.dtype != bf:
            return "weights that are not bfloat16"
        if a.position is not None and type(a.position) is not RotaryEmbedding:
            return "another position encoding"
        if a.hidden != H or f.hidden != H or a.q_dim % 8 or f.inter % 8 or a.head_dim > 512:
            return "sizes the chain does not take"
        for w in (a.w_qkv, a.w_o, f.w_gate_up, f.w_down):
            if w.stride(1) != 1 or w.stride(0) % 8 or w.data_ptr() % 16:
                return "a weight that is not aligned"
    return None


class ChainBuilder:
    """Collects operations, their tensor maps and the buffers between them."""

    def __init__(self, device, sms: Optional[int] = None):
        self.device = torch.device(device)
        self.sms = sms or torch.cuda.get_device_properties(self.device).multi_processor_count
        self._maps: list[bytes] = []
        self._map_of: dict = {}
        self._ops: list[list[int]] = []
        self._buffers: dict = {}
        self._keep: list = []               # tensors whose addresses the operations hold

    def __len__(self) -> int:
        return len(self._ops)

    def buffer(self, name: str, shape: tuple, dtype) -> torch.Tensor:
        """A zeroed buffer, shared by all who ask for the same name, shape and type."""
        key = (name, tuple(shape), dtype)
        t = self._buffers.get(key)
        if t is None:
            t = self._buffers[key] = torch.zeros(shape, dtype=dtype, device=self.device)
        return t

    def _map(self, t: torch.Tensor, box_rows: int) -> int:
        key = (t.data_ptr(), tuple(t.shape), t.stride(0), box_rows)
        idx = self._map_of.get(key)
        if idx is None:
            idx = self._map_of[key] = len(self._maps)
            self._maps.append(kernels.chain_make_map(t, box_rows))
            self._keep.append(t)
        return idx

    def _op(self, **fields) -> None:
        row = [0] * kernels.CHAIN_OP_FIELDS
        for k, v in fields.items():
            row[F[k]] = int(v)
        self._ops.append(row)

    def gemm(self, w: torch.Tensor, x: torch.Tensor, out, epi: int, activation: str = "gelu_tanh",
             cap: float = 0.0, max_split: int = MAX_SPLIT) -> torch.Tensor:
        """out = x w^T for x [16, K] bfloat16.  ``out``: a tensor, or the name of a float32 buffer
        [slices, 16, N] of partial sums made here (epilogue CHAIN_PARTS)."""
        gated = epi == kernels.CHAIN_GATED
        K = w.shape[1]
        N = w.shape[0] // 2 if gated else w.shape[0]
        assert x.shape == (ROWS, K) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
        row_tiles = (N + 63) // 64 if gated else (N + 127) // 128
        k_blocks = (K + 63) // 64
        slices, per = (1, k_blocks)
        if epi == kernels.CHAIN_PARTS:
            slices, per = choose_split(row_tiles, k_blocks, self.sms, max_split)
        if isinstance(out, str):
            out = self.buffer(out, (slices, ROWS, N), torch.float32)
        assert out.shape[-2:] == (ROWS, N) and out.stride(-1) == 1
        assert out.dtype == (torch.bfloat16 if gated else torch.float32)
        assert (out.dim() == 3 and out.shape[0] == slices) or slices == 1
        self._keep += [w, out]
        self._op(kind=kernels.CHAIN_GEMM, epi=epi, act=kernels.ACTIVATIONS[activation],
                 map_w=self._map(w, 64 if gated else 128), map_x=self._map(x, ROWS), N=N, K=K, ksplit=slices, per=per,
                 row_tiles=row_tiles, items=row_tiles * slices, ldy=out.stride(-2),
                 part_stride=out.stride(0) if out.dim() == 3 else 0, y=out.data_ptr(), cap=_bits(cap))
        return out

    def norm(self, h: torch.Tensor, parts: Optional[torch.Tensor], post: Optional[RMSNorm], nxt: Optional[RMSNorm],
             out: torch.Tensor) -> None:
        """h += post(sum of parts) (or the plain sum; nothing when parts is None); out = nxt(h)."""
        H = h.shape[1]
        assert h.dtype == torch.float32 and h.is_contiguous() and H % 8 == 0 and H <= MAX_HIDDEN
        assert parts is None or (parts.dim() == 3 and parts.shape[1:] == h.shape and parts.stride(1) == H)
        assert out.dtype == torch.bfloat16 and out.shape == h.shape and out.is_contiguous()
        self._keep += [h, parts, out, post.weight if post is not None else None, nxt.weight if nxt is not None else None]
        self._op(kind=kernels.CHAIN_NORM, h=h.data_ptr(), parts=parts.data_ptr() if parts is not None else 0,
                 n_parts=parts.shape[0] if parts is not None else 0,
                 in_stride=parts.stride(0) if parts is not None else 0, hidden=H,
                 w_post=post.weight.data_ptr() if post is not None else 0,
                 eps_post=_bits(post.eps if post is not None else 0.0),
                 off_post=_bits(post.offset if post is not None else 0.0),
                 w_next=nxt.weight.data_ptr() if nxt is not None else 0,
                 eps_next=_bits(nxt.eps if nxt is not None else 0.0),
                 off_next=_bits(nxt.offset if nxt is not None else 0.0), out=out.data_ptr())

    def rope(self, parts: torch.Tensor, out: torch.Tensor, table: Optional[torch.Tensor], rotary_dim: int, n_q: int,
             n_kv: int, head_dim: int, k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
             page_size: int, group: int) -> None:
        """out (bfloat16) = the sum of parts with q and k rotated; k and v also into the pages of ``group``."""
        width = (n_q + 2 * n_kv) * head_dim
        assert parts.dim() == 3 and parts.shape[1:] == (ROWS, width) and parts.stride(1) == width
        assert out.shape == (ROWS, width) and out.dtype == torch.bfloat16 and out.is_contiguous()
        assert n_q < 65536 and n_kv < 65536 and rotary_dim < 65536 and page_size < 65536 and 0 <= group < 4
        assert rotary_dim % 2 == 0 and rotary_dim <= head_dim and head_dim % 2 == 0
        self._keep += [parts, out, table, k_pages, v_pages]
        self._op(kind=kernels.CHAIN_ROPE, parts=parts.data_ptr(), n_parts=parts.shape[0], in_stride=parts.stride(0),
                 out=out.data_ptr(), cos_sin=table.data_ptr() if table is not None else 0,
                 k_pages=k_pages.data_ptr() if k_pages is not None else 0,
                 v_pages=v_pages.data_ptr() if v_pages is not None else 0,
                 heads=n_q | (n_kv << 16) | (head_dim << 32), rope=rotary_dim | (page_size << 16) | (group << 32))

    def finish(self) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(maps, ops, sync) on the device, as ``kernels.decode_chain`` takes them."""
        maps = torch.frombuffer(bytearray(b"".join(self._maps) or bytes(kernels.CHAIN_MAP_BYTES)),
                                dtype=torch.uint8).reshape(-1, kernels.CHAIN_MAP_BYTES).to(self.device)
        ops = torch.tensor(self._ops, dtype=torch.int64).reshape(-1, kernels.CHAIN_OP_FIELDS).to(self.device)
        return maps, ops, torch.zeros(4, dtype=torch.int32, device=self.device)


class DecodeChains:
    """The compiled decode step of one (model, cache).  The cache itself is not kept: a plan dies with it."""

    def __init__(self, model, cache):
        self.model = model
        b = self.builder = ChainBuilder(model.device)
        lay = model.layout
        H, V = lay.embedding.hidden, lay.embedding.vocab
        sched = lay.schedule
        self.entries = [cache.entries[i if c.cache_of is None else c.cache_of] for i, c in enumerate(sched)]
        if max(e.group_id for e in self.entries) > 3:
            raise ValueError("decode chains: more than four key/value groups")
        self.h = b.buffer("h", (ROWS, H), torch.float32)
        self.logits = b.buffer("logits", (ROWS, V), torch.float32)
        x = b.buffer("x", (ROWS, H), torch.bfloat16)
        self.segments: list[tuple[int, int]] = []       # (first operation, count); attention i runs after segment i
        self.layers: list[dict] = []

        start = len(b)
        b.norm(self.h, None, None, model.blocks[sched[0].block].pre_mixer_norm, x)
        self._mixer_in(0, x)
        self.segments.append((start, len(b) - start))
        for i, call in enumerate(sched):
            blk = model.blocks[call.block]
            a, f = blk.mixer, blk.feedforward
            start = len(b)
            o_parts = b.gemm(a.w_o, self.layers[i]["attn_out"], "o_parts", kernels.CHAIN_PARTS)
            b.norm(self.h, o_parts, blk.post_mixer_norm, blk.pre_ffn_norm, x)
            act = b.buffer("act", (ROWS, f.inter), torch.bfloat16)
            b.gemm(f.w_gate_up, x, act, kernels.CHAIN_GATED, activation=f.activation)
            d_parts = b.gemm(f.w_down, act, "down_parts", kernels.CHAIN_PARTS)
            if i + 1 < len(sched):
                b.norm(self.h, d_parts, blk.post_ffn_norm, model.blocks[sched[i + 1].block].pre_mixer_norm, x)
                self._mixer_in(i + 1, x)
            else:
                b.norm(self.h, d_parts, blk.post_ffn_norm, model.final_norm, x)
                b.gemm(model.head, x, self.logits, kernels.CHAIN_SOFTCAP, cap=float(lay.head.softcap or 0.0))
            self.segments.append((start, len(b) - start))
        self.maps, self.ops, self.sync = b.finish()

    def _mixer_in(self, i: int, x: torch.Tensor) -> None:
        """The fused q/k/v product of schedule entry i, its rotation and the write into the cache."""
        b = self.builder
        call = self.model.layout.schedule[i]
        a: Attention = self.model.blocks[call.block].mixer
        entry = self.entries[i]
        parts = b.gemm(a.w_qkv, x, "qkv_parts", kernels.CHAIN_PARTS)
        qkv = b.buffer("qkv", (ROWS, a.q_dim + 2 * a.kv_dim), torch.bfloat16)
        attn_out = b.buffer("attn_out", (ROWS, a.q_dim), torch.bfloat16)
        writes = call.cache_of is None
        b.rope(parts, qkv, a.position.table if a.position is not None else None,
               a.position.rotary_dim if a.position is not None else 0, a.n_q, a.n_kv, a.head_dim,
               entry.k if writes else None, entry.v if writes else None, entry.group.page_size, entry.group_id)
        self.layers.append({"mixer": a, "entry": entry, "qkv": qkv, "attn_out": attn_out})

    def run(self, ctx, tokens: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        M = ctx.n_tokens
        lay = self.model.layout
        kernels.embed_scale(tokens, self.model.embedding, lay.embedding.scale, self.h[:M])
        cache_rows = list(ctx.cache_rows)
        for i, (first, count) in enumerate(self.segments):
            kernels.decode_chain(self.maps, self.ops, first, count, M, ctx.positions, cache_rows, self.sync)
            if i < len(self.layers):
                L = self.layers[i]
                a: Attention = L["mixer"]
                k_pages, v_pages, table, ring, page = ctx.kv(L["entry"])
                common = dict(n_kv=a.n_kv, group=a.n_q // a.n_kv, head_dim=a.head_dim, scale=a.scale, cap=a.softcap,
                              window=a.window or 0, batch=ctx.batch, max_q_len=ctx.max_q_len)
                a.attend_paged(L["qkv"][:M, :a.q_dim], L["attn_out"][:M], ctx, common, k_pages, v_pages, table, ring,
                               page)
        logits = self.logits[:M]
        if rows.numel() != M:
            return logits.index_select(0, rows.to(torch.long))
        if torch.cuda.is_current_stream_capturing():
            return logits                       # a captured step's result lives in the graph's own memory anyway
        return logits.clone()                   # the buffer is written again by the next step
