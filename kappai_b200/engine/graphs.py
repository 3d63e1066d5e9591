"""CUDA graphs for decode steps.

A decode step (every segment one token, every token's logits wanted) launches
about a hundred small kernels; from Python that is launch-bound.  Such a step
is captured once per shape into a CUDA graph whose kernels read the step's
tables (token ids, positions, slots, block tables) from a static device buffer;
later steps of the same shape only refill that buffer (one pinned-memory copy)
and replay.  The shape key is (number of requests, block-table width), the
width being the next power of two of the blocks needed, so a graph is captured
again only when the longest request doubles its pages.  The split-KV attention
grid is fixed by that width.  Nothing else differs from the eager path: the same
model code runs under capture.
"""
from __future__ import annotations

import gc
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..ops import kernels as K
from .batch import PagedView, StepContext, StepSegments, _Tables, upload_step

N_PINNED = 4          # staging buffers in rotation, so a refill never overtakes a copy in flight


def _align4(n: int) -> int:
    return (n + 3) // 4 * 4


class _DecodeGraph:
    def __init__(self, runner, n: int, width: int):
        self.n, self.width = n, width
        dev = runner.device
        groups = list(runner.group_page_size.items())
        # layout of the static buffer (int32), every piece 16-byte aligned
        off, self.off = 0, {}
        for name in ("token_ids", "positions", "row_seg", "cu_rows", "seg_pos", "seg_slot", "logit_rows"):
            self.off[name] = off
            off += _align4(n + 1 if name == "cu_rows" else n)
        for gk, _ in groups:
            self.off[("slot_map", gk)] = off
            off += _align4(n)
            self.off[("block_table", gk)] = off
            off += _align4(n * width)
        # tables of their own that parts build for every step: laid out once from a step of this shape (their
        # sizes may depend on the number of requests only) and refilled before every replay
        self.builders = dict(runner.model.table_builders)
        self.part_layout = {}                      # key -> ([(name, offset, size)], scalars)
        segs0 = self._segments([0] * n)
        for key, b in self.builders.items():
            t = b.step_tables(segs0)
            if t is None:
                continue
            pieces = []
            for name, arr in t.arrays.items():
                arr = np.asarray(arr, dtype=np.int32).reshape(-1)
                pieces.append((name, off, arr.size))
                off += _align4(arr.size)
            self.part_layout[key] = (pieces, dict(t.scalars))
        self.size = off
        self.dev = torch.zeros(off, dtype=torch.int32, device=dev)
        self.pinned = [torch.zeros(off, dtype=torch.int32, pin_memory=True) for _ in range(N_PINNED)]
        self.pinned_np = [p.numpy() for p in self.pinned]
        self.events = [None] * N_PINNED
        self.turn = 0
        # The tables are kept in one host array and changed in place from step to step (a block-table row is
        # rewritten only when its request or the request's table has changed); each step copies the array
        # to the next staging buffer.
        self.host = np.zeros(off, dtype=np.int32)
        a = self.host                               # the pieces that never change
        a[self.off["row_seg"]:self.off["row_seg"] + n] = np.arange(n)
        a[self.off["cu_rows"]:self.off["cu_rows"] + n + 1] = np.arange(n + 1)
        a[self.off["logit_rows"]:self.off["logit_rows"] + n] = np.arange(n)
        self.host_bt = {gk: a[self.off[("block_table", gk)]:self.off[("block_table", gk)] + n * width].reshape(n, width)
                        for gk, _ in groups}
        self.host_sm = {gk: a[self.off[("slot_map", gk)]:self.off[("slot_map", gk)] + n] for gk, _ in groups}
        self.row_key = {gk: [None] * n for gk, _ in groups}     # (request, table version) a row was written for
        piece = lambda name, m: self.dev[self.off[name]:self.off[name] + m]
        paged = {gk: PagedView(piece(("block_table", gk), n * width).view(n, width), piece(("slot_map", gk), n), ps)
                 for gk, ps in groups}
        max_ctx = min(runner.max_model_len, width * runner.page_size)
        self.ctx = StepContext(
            n_rows=n, n_seg=n, token_ids=piece("token_ids", n), positions=piece("positions", n),
            row_seg=piece("row_seg", n), cu_rows=piece("cu_rows", n + 1), seg_pos=piece("seg_pos", n),
            seg_slot=piece("seg_slot", n), logit_rows=piece("logit_rows", n), n_out=n, paged=paged,
            host_cu_rows=list(range(n + 1)), host_seg_pos=[0] * n, host_seg_slot=[0] * n,
            max_seg_len=1, max_context=max_ctx, decode_only=True,
            tables={key: _Tables(**{name: self.dev[o:o + m] for name, o, m in pieces}, **scalars)
                    for key, (pieces, scalars) in self.part_layout.items()})
        self.ctx.h2d_bytes = off * 4
        self.last_used = 0
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.n_kernels = 0

    def _segments(self, lens) -> StepSegments:
        n = self.n
        return StepSegments(n, n, np.arange(n + 1, dtype=np.int32), np.asarray(lens, dtype=np.int32), [1] * n, 1, True)

    def _fill_part_tables(self, lens) -> None:
        segs = self._segments(lens)
        for key, (pieces, scalars) in self.part_layout.items():
            t = self.builders[key].step_tables(segs)
            if t is None or dict(t.scalars) != scalars or set(t.arrays) != {p[0] for p in pieces}:
                raise RuntimeError(f"step tables {key!r}: a captured decode step needs the same tables every step")
            for name, o, m in pieces:
                arr = np.asarray(t.arrays[name], dtype=np.int32).reshape(-1)
                if arr.size != m:
                    raise RuntimeError(f"step tables {key!r}: '{name}' changed its size in a captured decode step")
                self.host[o:o + m] = arr

    def fill(self, runner, reqs: Sequence[Hashable], tokens: Optional[Sequence[int]],
             device_tokens: Optional[torch.Tensor] = None) -> None:
        """Write this step's tables into the next staging buffer and bring them to the device (a kernel reads the
        pinned buffer: cheaper between two graph launches than a copy engine's 2 KB), with ``device_tokens`` in
        the tokens' place if given."""
        i = self.turn
        self.turn = (i + 1) % N_PINNED
        if self.events[i] is not None:
            self.events[i].synchronize()
        a = self.host
        n, o = self.n, self.off
        cache = runner.cache
        rcs = [cache.requests[r] for r in reqs]
        lens = [rc.length for rc in rcs]
        if tokens is not None:
            a[o["token_ids"]:o["token_ids"] + n] = tokens
        a[o["positions"]:o["positions"] + n] = lens
        a[o["seg_pos"]:o["seg_pos"] + n] = lens
        a[o["seg_slot"]:o["seg_slot"] + n] = [rc.slot for rc in rcs]
        for gk, ps in runner.group_page_size.items():
            pool = cache.pools[gk]
            bt, sm, keys = self.host_bt[gk], self.host_sm[gk], self.row_key[gk]
            for j, r in enumerate(reqs):
                t = pool.table(r)
                key = (r, pool.version(r))
                if keys[j] != key:
                    bt[j, :len(t)] = t
                    bt[j, len(t):] = 0
                    keys[j] = key
                sm[j] = t[lens[j] // ps] * ps + lens[j] % ps
        if self.part_layout:
            self._fill_part_tables(lens)
        np.copyto(self.pinned_np[i], a)
        K.step_tables(self.pinned[i], self.dev, device_tokens, self.off["token_ids"])
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class _StepGraph:
    """A captured step of any shape (prompt portions, portions beside decoded tokens): its tables live in one static
    device buffer, laid out as :func:`~kappai_b200.engine.batch.lay_out_step` lays them out; a later step with
    the same signature brings its tables there and replays."""

    def __init__(self, runner, host):
        self.dev = torch.zeros(host.flat.size, dtype=torch.int32, device=runner.device)
        self.pinned = [torch.zeros(host.flat.size, dtype=torch.int32, pin_memory=True) for _ in range(N_PINNED)]
        self.pinned_np = [p.numpy() for p in self.pinned]
        self.events = [None] * N_PINNED
        self.turn = 0
        self.ctx = upload_step(host, runner.device, into=self.dev)
        self.last_used = 0
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.n_kernels = 0

    def fill(self, host, device_tokens: Optional[torch.Tensor] = None) -> None:
        i = self.turn
        self.turn = (i + 1) % N_PINNED
        if self.events[i] is not None:
            self.events[i].synchronize()
        np.copyto(self.pinned_np[i], host.flat)
        K.step_tables(self.pinned[i], self.dev, device_tokens, host.offs[0])
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class DecodeGraphs:
    """Captured decode steps of one :class:`ModelRunner`."""

    def __init__(self, runner):
        self.runner = runner
        self.graphs: Dict[Tuple[int, int], _DecodeGraph] = {}
        self.seen: Dict[Tuple[int, int], int] = {}     # how often a shape has come without being captured
        self.step_graphs: Dict[tuple, _StepGraph] = {}   # captured steps of other shapes, by their tables' signature
        self.step_last, self.step_run = None, 0          # the signature of the last such step, and how often in a row
        self.n_step_captures = 0
        self.pool = None                               # the captures' shared memory pool
        self.capture_stream = None                     # the stream that captures run on
        self.clock = 0                                 # counts the steps: a graph remembers when it last ran
        self.n_evicted = 0
        self.n_captures = 0
        self.n_replays = 0

    # A shape (requests, table width) is captured when it comes for the second time: a capture costs several
    # steps' time, and under load the number of requests changes from step to step (requests end one by one), so
    # most shapes are seen once and never again; those run kernel by kernel.
    CAPTURE_AFTER = 2
    # Captured graphs share one memory pool (what a capture frees, the next may use) and at most MAX_GRAPHS are
    # kept: beyond that the one that was replayed longest ago goes.  Each keeps its activations and an
    # n x vocabulary logits buffer alive (16 MB at 64 requests and a vocabulary of 65536).
    MAX_GRAPHS = 64

    @staticmethod
    def eligible(entries) -> bool:
        return all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)

    def wants(self, entries) -> bool:
        """Should this decode step run from a captured graph (one that exists, or one that is due)?"""
        r = self.runner
        blocks = 1
        for e in entries:
            rc = r.cache.requests.get(e.req)
            need = (rc.length if rc is not None else 0) + 1
            for ps in r.group_page_size.values():
                blocks = max(blocks, -(-need // ps))
        key = (len(entries), self.width_for(blocks))
        g = self.graphs.get(key)
        if g is not None and g.graph is not None:
            return True
        self.seen[key] = self.seen.get(key, 0) + 1
        return self.seen[key] >= self.CAPTURE_AFTER

    def width_for(self, blocks: int) -> int:
        w = 8
        while w < blocks:
            w *= 2
        return w

    def step(self, entries, device_tokens: Optional[torch.Tensor]) -> torch.Tensor:
        """Pages for the new tokens are already taken.  Returns the static
        logits buffer [n, vocab] (valid until the next step of this shape)."""
        r = self.runner
        reqs = [e.req for e in entries]
        n = len(reqs)
        blocks = max(len(r.cache.block_table(q, gk)) for q in reqs for gk in r.group_page_size) \
            if r.group_page_size else 1
        key = (n, self.width_for(blocks))
        g = self.graphs.get(key)
        if g is None:
            g = _DecodeGraph(r, n, key[1])
            self.graphs[key] = g
        self.clock += 1
        g.last_used = self.clock
        tokens = None if device_tokens is not None else [int(e.tokens[0]) for e in entries]
        g.fill(r, reqs, tokens, device_tokens)
        if g.graph is None:
            # run once eagerly (kernels get built, scratch gets its size), restore the state it changed, capture
            self._capture(g)
        else:
            g.graph.replay()
            K.LAUNCHES[0] += g.n_kernels
            self.n_replays += 1
        r.last_h2d_bytes = g.ctx.h2d_bytes
        return g.logits

    # Steps that are not pure decode (a prompt portion, portions beside decoded tokens) launch some 130 kernels
    # from Python, about 2 ms of host time, which is more than the device needs for less than a thousand rows.
    # Where the same shape comes again -- a long prompt fed in equal portions, beside the same decoding requests --
    # the step is captured like a decode step: by its tables' signature, with the block tables' width and the
    # largest context rounded up so that the signature holds while the prompt grows.
    # Measured (LFM2-1.2B shape, 8 decoded tokens beside a prompt portion): 72 rows 2.19 -> 1.36 ms a step, 264 rows
    # 2.29 -> 2.04 ms (there the device itself needs 2 ms); a capture costs about 23 ms.
    STEP_MAX_ROWS = 160            # larger steps keep the device busy for about as long as the host needs to launch them
    STEP_CAPTURE_AFTER = 3         # times in a row: the shape must look like staying

    def round_blocks(self, blocks: int) -> int:
        return self.width_for(blocks)

    @staticmethod
    def round_context(tokens: int) -> int:
        c = 2048
        while c < tokens:
            c *= 2
        return c

    def wants_step(self, host) -> bool:
        """Should this step run from a captured graph: one that exists, or one that is due because the same shape
        has now come STEP_CAPTURE_AFTER times in a row (a shape that merely comes back now and then, like a
        prompt of some length, is not worth a capture)."""
        if host.n_rows > self.STEP_MAX_ROWS:
            self.step_last, self.step_run = None, 0
            return False
        key = host.signature()
        self.step_run = self.step_run + 1 if key == self.step_last else 1
        self.step_last = key
        g = self.step_graphs.get(key)
        return (g is not None and g.graph is not None) or self.step_run >= self.STEP_CAPTURE_AFTER

    def run_step(self, host, device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run a laid-out step from its captured graph (captured now if it is not yet).  Returns the static logits
        buffer (valid until the next step of this signature), None if the step wants none."""
        r = self.runner
        key = host.signature()
        g = self.step_graphs.get(key)
        if g is None:
            g = _StepGraph(r, host)
            self.step_graphs[key] = g
        self.clock += 1
        g.last_used = self.clock
        g.fill(host, device_tokens)
        if g.graph is None:
            self._capture(g)
        else:
            g.graph.replay()
            K.LAUNCHES[0] += g.n_kernels
            self.n_replays += 1
        r.last_h2d_bytes = g.ctx.h2d_bytes
        return g.logits

    def _capture(self, g) -> None:
        r = self.runner
        # the eager warm-up run changes fixed-size state (and rewrites this step's keys, harmlessly);
        # keep a copy of the state tensors and put them back before the captured run replays the step
        from ..cache.storage import StateView
        states = [v.tensor for v in r.storage.views if isinstance(v, StateView) and v.writes]
        saved = [t.clone() for t in states]
        torch.cuda.current_stream().synchronize()
        r.model.forward(g.ctx, r.storage.views)
        for t, s in zip(states, saved):
            t.copy_(s)
        torch.cuda.current_stream().synchronize()
        graph = torch.cuda.CUDAGraph()
        before = K.LAUNCHES[0]
        # Python's cycle collector must not run inside the capture: a dead cycle may hold captured graphs of
        # an engine that is gone, and destroying a CUDA graph while a stream captures invalidates the capture.
        # So the collector rests until the capture has ended.  The capture is begun and ended by hand, on a
        # stream of its own: torch.cuda.graph() would first synchronise the device, run a full collection and
        # empty the allocator's cache, which is most of the 40 to 100 ms that a capture took with it.
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            if self.pool is None:
                self.pool = torch.cuda.graph_pool_handle()
            if self.capture_stream is None:
                self.capture_stream = torch.cuda.Stream()
            cur = torch.cuda.current_stream()
            self.capture_stream.wait_stream(cur)
            with torch.cuda.stream(self.capture_stream):
                graph.capture_begin(pool=self.pool)
                try:
                    g.logits = r.model.forward(g.ctx, r.storage.views)
                finally:
                    graph.capture_end()
            cur.wait_stream(self.capture_stream)
        finally:
            if gc_was_on:
                gc.enable()
        g.n_kernels = K.LAUNCHES[0] - before       # kernel launchers a replay stands for
        for t, s in zip(states, saved):
            t.copy_(s)
        g.graph = graph
        if isinstance(g, _StepGraph):
            self.n_step_captures += 1
        else:
            self.n_captures += 1
        captured = [(d, k) for d in (self.graphs, self.step_graphs) for k, v in d.items() if v.graph is not None]
        if len(captured) > self.MAX_GRAPHS:
            # (no kernel of the oldest graph can still be running behind the replays that came after it on this stream)
            d, oldest = min(((d, k) for d, k in captured if d[k] is not g), key=lambda dk: dk[0][dk[1]].last_used)
            torch.cuda.current_stream().synchronize()
            del d[oldest]
            self.seen.pop(oldest, None)
            self.n_evicted += 1
        graph.replay()
        self.n_replays += 1
