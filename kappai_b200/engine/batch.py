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
    # tables that parts asked for through ``step_tables`` (see parts.base.Part): key -> namespace whose
    # attributes are the part's int32 arrays on the device and its host scalars
    tables: Dict[Hashable, object] = field(default_factory=dict)


@dataclass
class StepSegments:
    """The host's view of a step's segments, handed to the parts' ``step_tables``."""

    n_rows: int
    n_seg: int
    cu_rows: np.ndarray            # int32 [n_seg + 1]
    seg_pos: np.ndarray            # int32 [n_seg]
    seg_len: List[int]
    max_seg_len: int
    decode_only: bool


@dataclass
class PartTables:
    """What a part's ``step_tables`` returns: int32 arrays that go to the device with the step's one upload,
    and host values (sizes, counts) that stay on the host."""

    arrays: Dict[str, np.ndarray] = field(default_factory=dict)
    scalars: Dict[str, int] = field(default_factory=dict)


class _Tables:
    """Attribute access to one part's tables of a step."""

    def __init__(self, **kw):
        self.__dict__.update(kw)


@dataclass
class HostStep:
    """A step's tables laid out on the host: one int32 array of 16-byte aligned pieces, and where each piece is."""

    flat: np.ndarray                                   # int32, all pieces
    offs: List[int]                                    # first word of piece i
    sizes: List[int]                                   # words of piece i
    n_rows: int
    n_seg: int
    n_out: int
    host_cu_rows: List[int]
    host_seg_pos: List[int]
    host_seg_slot: List[int]
    max_seg_len: int
    max_context: int
    decode_only: bool
    paged: Dict[Hashable, tuple]                       # group -> (index of its block-table piece, its shape, page size)
    part_tables: list                                  # (key, [(name, index of the piece)], scalars)

    def signature(self) -> tuple:
        """Everything that a launch of the step may depend on beside the tables' contents: two steps with the same
        signature launch the same kernels with the same arguments, given the same addresses."""
        return (self.n_rows, self.n_seg, self.n_out, self.max_seg_len, self.max_context, self.decode_only,
                tuple(self.sizes), tuple((gk, shape) for gk, (_, shape, _) in self.paged.items()),
                tuple((key, tuple(sorted(sc.items()))) for key, _, sc in self.part_tables))


def build_step_context(segments: Sequence[Segment], groups: Dict[Hashable, int], device: torch.device,
                       vocab_size: int, max_positions: int, table_builders: Optional[Dict[Hashable, object]] = None
                       ) -> StepContext:
    """Validate the segments on the host and upload their tables in one copy."""
    return upload_step(lay_out_step(segments, groups, vocab_size, max_positions, table_builders), device)


def lay_out_step(segments: Sequence[Segment], groups: Dict[Hashable, int], vocab_size: int, max_positions: int,
                 table_builders: Optional[Dict[Hashable, object]] = None, round_blocks=None, round_context=None
                 ) -> HostStep:
    """Validate the segments and lay their tables out on the host.

    ``round_blocks`` / ``round_context`` (for steps that may be captured): the width of the block tables and the
    step's largest context are rounded up by them, so that steps that differ a little share a signature.

    ``groups`` maps each page group to its page size.  Everything that could
    make a kernel read or write out of bounds is refused here, before any
    launch (token ids: src/context.c:866-867; positions: src/context.c:998-999).
    ``table_builders`` maps a key to a part whose ``step_tables(StepSegments)``
    adds tables of its own to the upload (tile lists, scan boundaries, ...).
    """
    if not segments:
        raise BatchError("a step needs at least one segment")
    seen = set()
    n_rows = 0
    token_arrays = []
    for s in segments:
        if s.req in seen:
            raise BatchError(f"request {s.req!r} appears twice in one step")
        seen.add(s.req)
        if len(s.tokens) < 1:
            raise BatchError(f"request {s.req!r}: a segment needs at least one token")
        if s.pos_start < 0 or s.pos_start + len(s.tokens) > max_positions:
            raise BatchError(f"request {s.req!r}: positions {s.pos_start}..{s.pos_start + len(s.tokens) - 1} "
                             f"exceed the engine's limit of {max_positions}")
        ids = np.asarray(s.tokens, dtype=np.int64)
        if ids.min() < 0 or ids.max() >= vocab_size:
            t = int(ids[(ids < 0) | (ids >= vocab_size)][0])
            raise BatchError(f"request {s.req!r}: token id {t} outside the vocabulary of {vocab_size}")
        token_arrays.append(ids)
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
        token_ids[r:r + n] = token_arrays[i]
        positions[r:r + n] = np.arange(s.pos_start, s.pos_start + n)
        row_seg[r:r + n] = i
        seg_pos[i], seg_slot[i] = s.pos_start, s.slot
        logit_rows.extend(r + int(w) for w in s.want)
        r += n
        cu_rows[i + 1] = r
    if len(set(seg_slot.tolist())) != n_seg:
        raise BatchError("two segments of one step name the same state slot")

    parts = [token_ids, positions, row_seg, cu_rows, seg_pos, seg_slot, np.asarray(logit_rows, dtype=np.int32)]
    seg_len = [len(s.tokens) for s in segments]
    host_segs = StepSegments(n_rows, n_seg, cu_rows, seg_pos, seg_len, max(seg_len), all(n == 1 for n in seg_len))
    part_tables = []                                   # (key, [(name, index into parts)], scalars)
    for key, builder in (table_builders or {}).items():
        t = builder.step_tables(host_segs)
        if t is None:
            continue
        names = []
        for name, arr in t.arrays.items():
            names.append((name, len(parts)))
            parts.append(np.ascontiguousarray(arr, dtype=np.int32).reshape(-1))
        part_tables.append((key, names, dict(t.scalars)))
    paged_host = {}
    for gk, page_size in groups.items():
        max_blocks = max(1, max(len(s.block_tables.get(gk, ())) for s in segments))
        if round_blocks is not None:
            max_blocks = int(round_blocks(max_blocks))
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

    sizes = [int(p.size) for p in parts]
    offs = np.concatenate([[0], np.cumsum([(s + 3) // 4 * 4 for s in sizes])])     # 16-byte aligned pieces
    flat = np.zeros(int(offs[-1]), dtype=np.int32)
    for p, o in zip(parts, offs[:-1]):
        flat[o:o + p.size] = p
    max_context = max(s.pos_start + len(s.tokens) for s in segments)
    if round_context is not None:
        max_context = int(round_context(max_context))
    return HostStep(flat=flat, offs=[int(o) for o in offs[:-1]], sizes=sizes, n_rows=n_rows, n_seg=n_seg,
                    n_out=len(logit_rows), host_cu_rows=cu_rows.tolist(), host_seg_pos=seg_pos.tolist(),
                    host_seg_slot=seg_slot.tolist(), max_seg_len=host_segs.max_seg_len, max_context=max_context,
                    decode_only=host_segs.decode_only, paged=paged_host, part_tables=part_tables)


def upload_step(host: HostStep, device: torch.device, into: Optional[torch.Tensor] = None) -> StepContext:
    """The device's view of a laid-out step.  Without ``into`` the tables travel now, in one copy from pinned
    memory; with it (an int32 device buffer as long as ``host.flat``) the context's tensors are views of that
    buffer and the caller brings the tables there (a captured step: the same buffer every time)."""
    if into is None:
        flat = torch.empty(host.flat.size, dtype=torch.int32, pin_memory=device.type == "cuda")
        flat.numpy()[:] = host.flat
        dev = flat.to(device, non_blocking=True)
    else:
        if into.dtype != torch.int32 or into.numel() != host.flat.size:
            raise BatchError("upload_step: the buffer does not fit the step's tables")
        flat, dev = None, into
    offs, sizes = host.offs, host.sizes
    piece = lambda i: dev[offs[i]:offs[i] + sizes[i]]

    paged = {}
    for gk, (i, shape, page_size) in host.paged.items():
        paged[gk] = PagedView(piece(i).view(shape), piece(i + 1), page_size)
    tables = {key: _Tables(**{name: piece(i) for name, i in names}, **scalars)
              for key, names, scalars in host.part_tables}
    ctx = StepContext(
        n_rows=host.n_rows, n_seg=host.n_seg, token_ids=piece(0), positions=piece(1), row_seg=piece(2), cu_rows=piece(3),
        seg_pos=piece(4), seg_slot=piece(5), logit_rows=piece(6), n_out=host.n_out, paged=paged,
        host_cu_rows=host.host_cu_rows, host_seg_pos=host.host_seg_pos, host_seg_slot=host.host_seg_slot,
        max_seg_len=host.max_seg_len, max_context=host.max_context,
        decode_only=host.decode_only, tables=tables)
    ctx._pinned = flat          # keep the pinned buffer alive until the copy has run
    ctx.h2d_bytes = host.flat.size * 4
    return ctx
