"""Turns the segments of one step into ONE flat int32 buffer in pinned host memory,
uploads it with one copy, and hands the model typed device views of it.

A segment is (request cache, its next tokens, the position of the first of them,
which of them want logits).  Segments of one token go to the decode work list,
longer ones are cut into tiles of 128 query rows for the prefill kernels.  The buffer is
filled by the native host core (csrc/host_core.cpp) from the requests' own block tables.  The
buffer holds, in this order (sizes in int32 words; T tokens, S segments, R rows,
G cache groups, B block-table width, L tiles):

    token_ids[T] token_src[T] positions[T] seq_of_token[T]
    slots[G][T] block_table[G][S*B]
    state_slot[S] decode_info[S][4] tile_seq[L] tile_tok[L] tile_rows[L]
    logit_rows[R] temperature[R] top_k[R] top_p[R] seed_lo[R] seed_hi[R] sample_pos[R]

(the reference's layout: src/core/batch_builder.cpp:17-46; one upload:
src/cuda/engine/engine.cpp:267-278).  The layout depends only on the capacities
(T, S, R, L), so a fixed-shape decode batch has the same device addresses every
time and can be replayed as a CUDA graph.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache import native
from ..cache.manager import CacheManager, RequestCache

# The work lists of a step are cut for the mixers that read them: sequences that bring more than
# one token into tiles of ``tile_rows`` query rows, the context of a single token into partitions
# of ``partition`` keys.  The engine takes both numbers from its model's mixers (``Mixer.tiling``);
# these defaults serve a builder made without a model.
DEFAULT_TILE_ROWS = 128
DEFAULT_PARTITION = 128


@dataclass
class RowSampling:
    """Sampling parameters of one logits row (sampling/params.py: SamplingParams)."""

    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0


@dataclass
class Segment:
    cache: RequestCache
    tokens: Sequence[int]          # the segment's token ids (ignored where src_row >= 0)
    start_pos: int                 # position of tokens[0]
    want: Sequence[int] = ()       # indices into tokens whose logits are wanted
    src_row: int = -1              # >= 0: the single token is row src_row of the previous step's samples
    sampling: Optional[RowSampling] = None   # applies to every wanted row of the segment


@dataclass
class GroupView:
    slots: torch.Tensor         # [T] cache slot of every token in this group (-1: none)
    block_table: torch.Tensor   # [S, B]


class Layout:
    def __init__(self, T: int, S: int, R: int, L: int, G: int, B: int):
        self.T, self.S, self.R, self.L, self.G, self.B = T, S, R, L, G, B
        off = 0

        def take(n: int) -> int:
            nonlocal off
            o = off
            off += (n + 3) // 4 * 4      # every field starts on a 16-byte boundary
            return o

        self.token_ids = take(T)
        self.token_src = take(T)
        self.positions = take(T)
        self.seq_of_token = take(T)
        self.slots = [take(T) for _ in range(G)]
        self.block_table = [take(S * B) for _ in range(G)]
        self.state_slot = take(S)
        self.decode_info = take(4 * S)   # per decode item: token index, sequence index, context length, 0
        self.tile_seq = take(L)
        self.tile_tok = take(L)
        self.tile_rows = take(L)
        self.logit_rows = take(R)
        self.temperature = take(R)
        self.top_k = take(R)
        self.top_p = take(R)
        self.seed_lo = take(R)
        self.seed_hi = take(R)
        self.sample_pos = take(R)
        self.words = off
        self._native = None

    def native(self):
        """The offsets as the native host core takes them (and, beside, those of the per-group fields)."""
        if self._native is None:
            nl = native.RlLayout()
            for name, _ in native.RlLayout._fields_:
                setattr(nl, name, getattr(self, name))
            self._native = nl
            self.slots_c = (ctypes.c_int32 * max(self.G, 1))(*self.slots)
            self.tables_c = (ctypes.c_int32 * max(self.G, 1))(*self.block_table)
        return self._native


@dataclass
class StepContext:
    """Device views of one step's metadata plus the host numbers kernels need for
    their grids.  ``host`` keeps the numpy arrays for parts that work on the host side
    (test parts) and for debugging."""

    T: int
    S: int
    R: int
    num_decode: int
    num_tiles: int
    decode_parts: int        # partitions per decode item in this launch
    max_items: int           # capacity of the decode workspace in items
    parts_capacity: int      # capacity of the decode workspace in partitions per item
    token_ids: torch.Tensor
    token_src: torch.Tensor
    positions: torch.Tensor
    seq_of_token: torch.Tensor
    state_slot: torch.Tensor
    decode_info: torch.Tensor    # [S, 4]
    tile_seq: torch.Tensor
    tile_tok: torch.Tensor
    tile_rows: torch.Tensor
    logit_rows: torch.Tensor
    temperature: torch.Tensor
    top_k: torch.Tensor
    top_p: torch.Tensor
    seed_lo: torch.Tensor
    seed_hi: torch.Tensor
    sample_pos: torch.Tensor
    groups: List[GroupView]
    status: torch.Tensor
    has_src: bool = False
    any_sampling: bool = False
    # the single-token sequences' context lengths (new token included): the longest and their sum
    decode_max_ctx: int = 0
    decode_sum_ctx: int = 0
    host: Optional["HostBatch"] = None
    profiler: Optional[object] = None          # engine.profiler.OpProfiler while per-op profiling is on
    # a norm handed over between parts (parts.base.NormHandover); set and cleared by the block
    next_norm: Optional[object] = None         # the norm applied to the stream after the running part
    hand_in: Optional[object] = None           # what the part before left for the running part's norm
    hand_out: Optional[object] = None          # what the running part leaves
    block_next_norm: Optional[object] = None   # set by the model: the first norm of the block after this one
    block_hand: Optional[object] = None        # carried from a block's last part to the next block


@dataclass
class HostBatch:
    q_start: List[int] = field(default_factory=list)
    q_len: List[int] = field(default_factory=list)
    start_pos: List[int] = field(default_factory=list)
    state_slot: List[int] = field(default_factory=list)
    keys: List[object] = field(default_factory=list)


class BatchBuilder:
    def __init__(self, cache: CacheManager, max_tokens: int, max_seqs: int, max_rows: int,
                 max_seq_len: int, device: torch.device, tile_rows: int = DEFAULT_TILE_ROWS,
                 partition: int = DEFAULT_PARTITION):
        self.cache = cache
        self.tile_rows, self.partition = tile_rows, partition
        self.G = len(cache.groups)
        self.page_size = cache.page_size
        self.max_tokens, self.max_seqs, self.max_rows = max_tokens, max_seqs, max_rows
        self.max_seq_len = max_seq_len
        self.B = cache.blocks_for(max_seq_len)
        self.max_tiles = (max_tokens + tile_rows - 1) // tile_rows + max_seqs
        self.parts_capacity = (max_seq_len + partition - 1) // partition
        cap = Layout(max_tokens, max_seqs, max_rows, self.max_tiles, self.G, self.B)
        self.device = device
        self.capacity_words = cap.words
        on_gpu = device.type == "cuda"
        self.num_slots = 4
        self.host_bufs = [torch.zeros(cap.words, dtype=torch.int32, pin_memory=on_gpu) for _ in range(self.num_slots)]
        self.host_np = [b.numpy() for b in self.host_bufs]
        self.events = [torch.cuda.Event() if on_gpu else None for _ in range(self.num_slots)]
        self.used = [False] * self.num_slots
        self.dev_buf = torch.zeros(cap.words, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._turn = 0
        self._lib = native.lib()

    def _views(self, lay: Layout, dev: torch.Tensor, T: int, S: int, R: int, L: int) -> dict:
        def v(off, n):
            return dev[off:off + n]

        f32 = lambda off, n: dev[off:off + n].view(torch.float32)  # noqa: E731
        return dict(
            token_ids=v(lay.token_ids, lay.T), token_src=v(lay.token_src, lay.T),
            positions=v(lay.positions, lay.T), seq_of_token=v(lay.seq_of_token, lay.T),
            state_slot=v(lay.state_slot, lay.S), decode_info=v(lay.decode_info, 4 * lay.S).view(lay.S, 4),
            tile_seq=v(lay.tile_seq, lay.L), tile_tok=v(lay.tile_tok, lay.L), tile_rows=v(lay.tile_rows, lay.L),
            logit_rows=v(lay.logit_rows, lay.R), temperature=f32(lay.temperature, lay.R),
            top_k=v(lay.top_k, lay.R), top_p=f32(lay.top_p, lay.R), seed_lo=v(lay.seed_lo, lay.R),
            seed_hi=v(lay.seed_hi, lay.R), sample_pos=v(lay.sample_pos, lay.R),
            groups=[GroupView(v(lay.slots[g], lay.T), v(lay.block_table[g], lay.S * lay.B).view(lay.S, lay.B))
                    for g in range(self.G)],
        )

    def build(self, segments: Sequence[Segment], pad_to: int = 0) -> StepContext:
        """Fills a pinned buffer, uploads it, returns the context.  ``pad_to`` > 0 (only
        for steps of single tokens that all want their logits) pads the batch with dummy
        one-token sequences on page 0 up to that many, so the shape is fixed."""
        S_real = len(segments)
        T_real = sum(len(s.tokens) for s in segments)
        R_real = sum(len(s.want) for s in segments)
        if S_real == 0 or T_real == 0:
            raise ValueError("a step needs at least one token")
        if S_real > self.max_seqs or T_real > self.max_tokens or R_real > self.max_rows:
            raise ValueError(f"step of {T_real} tokens, {S_real} sequences, {R_real} logits rows exceeds the "
                             f"engine's limits ({self.max_tokens}, {self.max_seqs}, {self.max_rows})")
        ps = self.page_size
        tiles = []
        for si, s in enumerate(segments):
            n = len(s.tokens)
            if n > 1:
                tiles.append((si, n))
        L_real = sum((n + self.tile_rows - 1) // self.tile_rows for _, n in tiles)
        if pad_to:
            T = S = R = pad_to
            L = 0
        else:
            T, S, R, L = T_real, S_real, R_real, L_real
        lay = Layout(T, S, R, L, self.G, self.B)

        slot = self._turn % self.num_slots
        self._turn += 1
        if self.used[slot] and self.events[slot] is not None:
            self.events[slot].synchronize()
        h = self.host_np[slot]
        hb = HostBatch()
        # ---- the fields are filled by the native host core from the requests' own block tables
        rows = []
        tok_parts = []
        want_flat: List[int] = []
        t = 0
        to = 0
        dec_max = dec_sum = 0
        for s in segments:
            n = len(s.tokens)
            if n == 1:
                dec_max = max(dec_max, s.start_pos + 1)
                dec_sum += s.start_pos + 1
            sp = s.sampling
            fed = s.src_row >= 0
            if sp is not None:
                rows.append((s.cache.rid, s.start_pos, n, s.src_row, to, len(want_flat), len(s.want), 1,
                             sp.temperature, sp.top_p, sp.top_k, sp.seed & 0xFFFFFFFF, (sp.seed >> 32) & 0xFFFFFFFF))
            else:
                rows.append((s.cache.rid, s.start_pos, n, s.src_row, to, len(want_flat), len(s.want), 0,
                             0.0, 1.0, 0, 0, 0))
            if not fed and n > 0:
                tok_parts.append(s.tokens)
                to += n
            want_flat.extend(s.want)
            hb.q_start.append(t)
            hb.q_len.append(n)
            hb.start_pos.append(s.start_pos)
            hb.state_slot.append(s.cache.state_slot)
            hb.keys.append(s.cache.key)
            t += n
        segs = np.array(rows, dtype=native.SEGMENT_DTYPE)
        if len(tok_parts) == 1:
            tokens = np.asarray(tok_parts[0], dtype=np.int32)
        elif tok_parts:
            tokens = np.concatenate([np.asarray(x, dtype=np.int32) for x in tok_parts])
        else:
            tokens = np.zeros(1, dtype=np.int32)
        tokens = np.ascontiguousarray(tokens)
        want = np.asarray(want_flat if want_flat else [0], dtype=np.int32)
        nl = lay.native()
        res = (ctypes.c_int32 * 8)()
        code = self._lib.rl_hc_build(self.cache._h, h.ctypes.data, ctypes.byref(nl), lay.slots_c, lay.tables_c,
                                     self.G, self.B, S_real, segs.ctypes.data, tokens.ctypes.data, want.ctypes.data,
                                     self.max_seq_len, self.tile_rows, res)
        if code < 0:
            s = segments[res[5]]
            if code == -10:
                raise ValueError("empty segment")
            if code == -11:
                raise ValueError(f"request {s.cache.key!r} would reach position {res[6]}, beyond max_seq_len "
                                 f"{self.max_seq_len}")
            if code == -12:
                raise ValueError("a device-fed segment has exactly one token")
            if code == -13:
                raise ValueError(f"request {s.cache.key!r}: pages reserved for {res[6]} positions, "
                                 f"step needs {s.start_pos + len(s.tokens)}")
            if code == -14:
                raise ValueError(f"wanted index {res[6]} outside a segment of {len(s.tokens)} tokens")
            raise ValueError(f"request {s.cache.key!r} is not open in the cache manager ({code})")
        nd, li, max_ctx, has_src, any_sampling = res[0], res[1], res[2], bool(res[3]), bool(res[4])
        if pad_to:
            if nd != S_real or R_real != S_real or T_real != S_real:
                raise ValueError("only steps of single tokens that all want logits can be padded")
            self._lib.rl_hc_pad(h.ctypes.data, ctypes.byref(nl), S_real, pad_to)
            nd = pad_to
            decode_parts = self.parts_capacity
        else:
            decode_parts = (max_ctx + self.partition - 1) // self.partition
        dev = self.dev_buf
        if self.device.type == "cuda":
            dev[:lay.words].copy_(self.host_bufs[slot][:lay.words], non_blocking=True)
            self.events[slot].record()
            self.used[slot] = True
        else:
            dev[:lay.words].copy_(self.host_bufs[slot][:lay.words])
        views = self._views(lay, dev, T, S, R, L)
        return StepContext(T=T, S=S, R=R, num_decode=nd, num_tiles=li, decode_parts=decode_parts,
                           max_items=self.max_seqs, parts_capacity=self.parts_capacity, status=self.status,
                           has_src=has_src, any_sampling=any_sampling, decode_max_ctx=dec_max,
                           decode_sum_ctx=dec_sum, host=hb, **views)
