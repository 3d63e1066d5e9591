"""The batch of one step: segments, flattened rows and their device tables.

The reference describes a step's rows with ``row_desc`` in three disjoint
modes (src/recipe.h:403-415): one chunk of one session, n single tokens of n
sessions, or several chunks ("segments", src/recipe/exec.c:938-971), and every
position-dependent op loops over the segments (src/recipe/internal.h:294-335).
Here there is one mode: a list of segments, each the next tokens of one
request; a decoded token is a segment of length one.  All rows of all
segments run through every kernel launch together.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch


class BatchError(ValueError):
    pass


@dataclass
class Segment:
    """The next tokens of one request in this step."""

    req: Hashable
    tokens: Sequence[int]
    pos_start: int                 # position of tokens[0] in the request's sequence
    want: Sequence[int] = ()       # indices into ``tokens`` whose logits are wanted
    slot: int = 0                  # the request's state slot
    block_tables: Dict[Hashable, List[int]] = field(default_factory=dict)   # group -> logical block -> page
    token_slots: Dict[Hashable, List[int]] = field(default_factory=dict)    # group -> physical slot per token


@dataclass
class PagedView:
    """Device tables of one page group for this step."""

    block_table: torch.Tensor      # int32 [n_seg, max_blocks]; -1 where a page was released
    slot_map: torch.Tensor         # int32 [n_rows]: page * page_size + offset of each row's key/value
    page_size: int


@dataclass
class StepContext:
    """Everything a part may need to know about the rows it is given."""

    n_rows: int
    n_seg: int
    token_ids: torch.Tensor        # int32 [n_rows]
    positions: torch.Tensor        # int32 [n_rows]
    row_seg: torch.Tensor          # int32 [n_rows]: segment of each row
    cu_rows: torch.Tensor          # int32 [n_seg + 1]: first row of each segment
    seg_pos: torch.Tensor          # int32 [n_seg]: position of each segment's first row
    seg_slot: torch.Tensor         # int32 [n_seg]: state slot of each segment's request
    logit_rows: torch.Tensor       # int32 [n_out]: rows whose logits are wanted
    n_out: int
    paged: Dict[Hashable, PagedView]
    # host copies (plain lists) for parts written in Python
    host_cu_rows: List[int]
    host_seg_pos: List[int]
    host_seg_slot: List[int]
    max_seg_len: int
    max_context: int               # largest position + 1 in the batch
    decode_only: bool              # every segment has one row
    tile_seg: Optional[torch.Tensor] = None    # int32 [n_tiles]: segment of each tile of ROW_TILE consecutive rows
    tile_row0: Optional[torch.Tensor] = None   # int32 [n_tiles]: first row of each tile
    n_tiles: int = 0
    # the same in stretches of BIG_TILE rows, those that read the most keys first (a kernel that gives a CTA the
    # i-th and the i-th last of them gives every CTA about the same work)
    big_tile_seg: Optional[torch.Tensor] = None
    big_tile_row0: Optional[torch.Tensor] = None
    n_big_tiles: int = 0
    # A step that mixes decoded tokens with prompt portions: the leading segments of at most SHORT_SEG rows
    # (the scheduler puts decodes first) can go to a kernel made for single rows with long caches and the rest
    # to a tiled one.  n_short_rows / n_short_tiles: rows and ROW_TILE tiles of that lead (0 if the step is not
    # mixed in this way); the big tiles then list the other segments only.
    n_short_rows: int = 0
    n_short_tiles: int = 0


BIG_TILE = 128                     # rows of the larger tiles
SHORT_SEG = 4                      # rows up to which a segment counts as short (decoded tokens)
ROW_TILE = 64                      # rows of one segment that a tiled kernel (prefill attention) takes at a time


def build_step_context(segments: Sequence[Segment], groups: Dict[Hashable, int], device: torch.device,
                       vocab_size: int, max_positions: int) -> StepContext:
    """Validate the segments on the host and upload their tables in one copy.

    ``groups`` maps each page group to its page size.  Everything that could
    make a kernel read or write out of bounds is refused here, before any
    launch (token ids: src/context.c:866-867; positions: src/context.c:998-999).
    """
    if not segments:
        raise BatchError("a step needs at least one segment")
    seen = set()
    n_rows = 0
    for s in segments:
        if s.req in seen:
            raise BatchError(f"request {s.req!r} appears twice in one step")
        seen.add(s.req)
        if len(s.tokens) < 1:
            raise BatchError(f"request {s.req!r}: a segment needs at least one token")
        if s.pos_start < 0 or s.pos_start + len(s.tokens) > max_positions:
            raise BatchError(f"request {s.req!r}: positions {s.pos_start}..{s.pos_start + len(s.tokens) - 1} "
                             f"exceed the engine's limit of {max_positions}")
        for t in s.tokens:
            if not (0 <= int(t) < vocab_size):
                raise BatchError(f"request {s.req!r}: token id {t} outside the vocabulary of {vocab_size}")
        for w in s.want:
            if not (0 <= int(w) < len(s.tokens)):
                raise BatchError(f"request {s.req!r}: wanted index {w} outside its {len(s.tokens)} tokens")
        n_rows += len(s.tokens)
    n_seg = len(segments)

    token_ids = np.empty(n_rows, np.int32)
    positions = np.empty(n_rows, np.int32)
    row_seg = np.empty(n_rows, np.int32)
    cu_rows = np.zeros(n_seg + 1, np.int32)
    seg_pos = np.empty(n_seg, np.int32)
    seg_slot = np.empty(n_seg, np.int32)
    logit_rows: List[int] = []
    r = 0
    for i, s in enumerate(segments):
        n = len(s.tokens)
        token_ids[r:r + n] = np.asarray(s.tokens, dtype=np.int64)
        positions[r:r + n] = np.arange(s.pos_start, s.pos_start + n)
        row_seg[r:r + n] = i
        seg_pos[i], seg_slot[i] = s.pos_start, s.slot
        logit_rows.extend(r + int(w) for w in s.want)
        r += n
        cu_rows[i + 1] = r
    if len(set(seg_slot.tolist())) != n_seg:
        raise BatchError("two segments of one step name the same state slot")

    tile_seg, tile_row0 = [], []
    for i in range(n_seg):
        for r0 in range(int(cu_rows[i]), int(cu_rows[i + 1]), ROW_TILE):
            tile_seg.append(i)
            tile_row0.append(r0)
    n_short_seg = 0
    while n_short_seg < n_seg and len(segments[n_short_seg].tokens) <= SHORT_SEG:
        n_short_seg += 1
    if n_short_seg == n_seg or all(len(s.tokens) > SHORT_SEG for s in segments):
        n_short_seg = 0                                   # all short or none: one kernel takes the whole step
    n_short_rows = int(cu_rows[n_short_seg])
    big = []
    for i in range(n_short_seg, n_seg):
        for r0 in range(int(cu_rows[i]), int(cu_rows[i + 1]), BIG_TILE):
            last_pos = int(seg_pos[i]) + min(r0 + BIG_TILE, int(cu_rows[i + 1])) - int(cu_rows[i]) - 1
            big.append((-last_pos, i, r0))                # the further on, the more keys
    big.sort()
    parts = [token_ids, positions, row_seg, cu_rows, seg_pos, seg_slot,
             np.asarray(logit_rows, dtype=np.int32), np.asarray(tile_seg, dtype=np.int32),
             np.asarray(tile_row0, dtype=np.int32), np.asarray([b[1] for b in big], dtype=np.int32),
             np.asarray([b[2] for b in big], dtype=np.int32)]
    n_fixed = len(parts)
    paged_host = {}
    for gk, page_size in groups.items():
        max_blocks = max(1, max(len(s.block_tables.get(gk, ())) for s in segments))
        bt = np.full((n_seg, max_blocks), -1, np.int32)
        sm = np.empty(n_rows, np.int32)
        r = 0
        for i, s in enumerate(segments):
            t = s.block_tables.get(gk)
            ts = s.token_slots.get(gk)
            n = len(s.tokens)
            if t is None or ts is None or len(ts) != n:
                raise BatchError(f"request {s.req!r}: no block table / token slots for page group {gk!r}")
            need = -(-(s.pos_start + n) // page_size)
            if len(t) < need:
                raise BatchError(f"request {s.req!r}: block table covers {len(t)} blocks, {need} needed")
            bt[i, :len(t)] = t
            sm[r:r + n] = ts
            r += n
        paged_host[gk] = (len(parts), bt.shape, page_size)
        parts.append(bt.reshape(-1))
        parts.append(sm)

    sizes = [p.size for p in parts]
    offs = np.concatenate([[0], np.cumsum([(s + 3) // 4 * 4 for s in sizes])])     # 16-byte aligned pieces
    flat = torch.empty(int(offs[-1]), dtype=torch.int32, pin_memory=device.type == "cuda")
    fl = flat.numpy()
    for p, o in zip(parts, offs[:-1]):
        fl[o:o + p.size] = p
    dev = flat.to(device, non_blocking=True)
    piece = lambda i: dev[int(offs[i]):int(offs[i]) + sizes[i]]

    paged = {}
    for gk, (i, shape, page_size) in paged_host.items():
        paged[gk] = PagedView(piece(i).view(shape), piece(i + 1), page_size)
    ctx = StepContext(
        n_rows=n_rows, n_seg=n_seg, token_ids=piece(0), positions=piece(1), row_seg=piece(2), cu_rows=piece(3),
        seg_pos=piece(4), seg_slot=piece(5), logit_rows=piece(6), n_out=len(logit_rows), paged=paged,
        host_cu_rows=cu_rows.tolist(), host_seg_pos=seg_pos.tolist(), host_seg_slot=seg_slot.tolist(),
        max_seg_len=max(len(s.tokens) for s in segments),
        max_context=max(s.pos_start + len(s.tokens) for s in segments),
        decode_only=all(len(s.tokens) == 1 for s in segments),
        tile_seg=piece(7), tile_row0=piece(8), n_tiles=len(tile_seg),
        big_tile_seg=piece(9), big_tile_row0=piece(10), n_big_tiles=len(big),
        n_short_rows=n_short_rows, n_short_tiles=n_short_seg)
    ctx._pinned = flat          # keep the pinned buffer alive until the copy has run
    ctx.h2d_bytes = flat.numel() * 4
    return ctx
