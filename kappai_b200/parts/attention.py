"""Grouped-query attention over the paged cache.

``q,k,v = h Wq^T, h Wk^T, h Wv^T`` (run as one product against the rows
[Wq; Wk; Wv], as the reference does with ``--fuse qkv``, src/model.c:1440-1448);
optional per-head RMSNorm of q and k with one weight [head_dim] shared by the
heads, before the rotation (src/models/lfm.c:36-39); position encoding; keys and
values into the cache; causal softmax attention with ``scale`` over the keys
``max(0, p - window + 1) .. p`` (src/backend/cpu/scalar/core.c:383-433);
``out = attn Wo^T`` added to the residual (src/models/lfm.c:51,
src/recipe/builders.c:381).

Sizes and constants (params): hidden_size, num_heads, num_kv_heads, head_dim,
scale, qk_norm_eps (None: no q/k norm), window (None: all keys), position (a
``position`` PartSpec), bias.
"""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from ..cache.spec import PagedKVSpec
from ..config.schema import ConfigError, PartSpec
from ..ops import kernels as K
from ..ops.linear import linear
from .base import Part, WeightSpec, make_part, register_part


# Geometry of the attention kernels' work lists (built on the host for every step that has prompt portions).
ROW_TILE = 64              # rows of one segment that the mma.sync prefill kernel takes at a time
BIG_TILE = 128             # rows of the tcgen05 prefill kernel's tiles
SHORT_SEG = 4              # segments of at most this many rows count as decoded tokens: split-KV kernel


def attention_tiles(segs, split_ok: bool = True):
    """Work lists of the tiled prefill kernels for one step (``engine.batch.StepSegments`` in,
    ``engine.batch.PartTables`` out; None for a step of short segments only, which the split-KV kernel takes).

    ``tile_seg`` / ``tile_row0``: segment and first row of every stretch of ROW_TILE consecutive rows of a
    segment.  ``big_tile_seg`` / ``big_tile_row0``: the same in stretches of BIG_TILE rows, those that read the
    most keys first (a kernel that gives a CTA the i-th and the i-th last of them gives every CTA about the same
    work).  A step that mixes decoded tokens with prompt portions: the leading segments of at most SHORT_SEG
    rows (the scheduler puts decodes first) go to the split-KV kernel, made for single rows with long caches,
    and the rest to a tiled one; ``n_short_rows`` / ``n_short_tiles`` are the rows and ROW_TILE tiles of that
    lead (0 if the step is not mixed in this way), and the big tiles then list the other segments only."""
    from ..engine.batch import PartTables

    if split_ok and segs.max_seg_len <= SHORT_SEG:
        return None
    cu, n_seg = segs.cu_rows, segs.n_seg
    tile_seg, tile_row0 = [], []
    for i in range(n_seg):
        for r0 in range(int(cu[i]), int(cu[i + 1]), ROW_TILE):
            tile_seg.append(i)
            tile_row0.append(r0)
    n_short_seg = 0
    while n_short_seg < n_seg and segs.seg_len[n_short_seg] <= SHORT_SEG:
        n_short_seg += 1
    if n_short_seg == n_seg or all(n > SHORT_SEG for n in segs.seg_len):
        n_short_seg = 0                                   # all short or none: one kernel takes the whole step
    big = []
    for i in range(n_short_seg, n_seg):
        for r0 in range(int(cu[i]), int(cu[i + 1]), BIG_TILE):
            last_pos = int(segs.seg_pos[i]) + min(r0 + BIG_TILE, int(cu[i + 1])) - int(cu[i]) - 1
            big.append((-last_pos, i, r0))                # the further on, the more keys
    big.sort()
    i32 = lambda v: np.asarray(v, dtype=np.int32)
    return PartTables(
        arrays={"tile_seg": i32(tile_seg), "tile_row0": i32(tile_row0),
                "big_tile_seg": i32([b[1] for b in big]), "big_tile_row0": i32([b[2] for b in big])},
        scalars={"n_tiles": len(tile_seg), "n_big_tiles": len(big), "n_short_rows": int(cu[n_short_seg]),
                 "n_short_tiles": n_short_seg})


class Attention(Part):
    category = "mixer"
    graph_safe = True

    def __init__(self, params, env):
        super().__init__(params, env)
        self.d = int(self._p("hidden_size"))
        self.H = int(self._p("num_heads"))
        self.G = int(self._p("num_kv_heads"))
        self.hd = int(self._p("head_dim"))
        self.scale = float(self._p("scale"))
        eps = self._p("qk_norm_eps", None)
        self.qk_norm_eps: Optional[float] = None if eps is None else float(eps)
        self.window: Optional[int] = self._p("window", None)
        self.bias = bool(self._p("bias", False))
        if self.H < 1 or self.G < 1 or self.H % self.G:
            raise ConfigError(f"attention: num_heads={self.H} must be a multiple of num_kv_heads={self.G}")
        if self.hd % 16 or not (16 <= self.hd <= 256):
            raise ConfigError(f"attention: head_dim={self.hd} is not supported by the kernels "
                              "(a multiple of 16 from 16 to 256)")
        pos = self._p("position", None)
        if pos is None:
            pos = PartSpec("none")
        elif isinstance(pos, dict):
            pos = PartSpec(**pos)
        self.position = make_part("position", pos, env)
        self.graph_safe = bool(self.position.graph_safe)     # a position part that reads host values keeps it eager
        self.split_ok = self.H // self.G <= K.SPLIT_MAX_RATIO
        self.step_tables_key = ("attention_tiles", self.split_ok)

    def step_tables(self, segs):
        return attention_tiles(segs, self.split_ok)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        d, H, G, hd = self.d, self.H, self.G, self.hd
        s = {"q_proj.weight": WeightSpec((H * hd, d)), "k_proj.weight": WeightSpec((G * hd, d)),
             "v_proj.weight": WeightSpec((G * hd, d)), "out_proj.weight": WeightSpec((d, H * hd))}
        if self.qk_norm_eps is not None:
            s["q_norm.weight"] = WeightSpec((hd,), "norm")
            s["k_norm.weight"] = WeightSpec((hd,), "norm")
        if self.bias:
            for n, sz in (("q_proj", H * hd), ("k_proj", G * hd), ("v_proj", G * hd), ("out_proj", d)):
                s[n + ".bias"] = WeightSpec((sz,), "bias")
        return s

    def bind(self, w):
        self.w_qkv = torch.cat([w["q_proj.weight"], w["k_proj.weight"], w["v_proj.weight"]], 0).contiguous()
        self.w_o = w["out_proj.weight"].contiguous()
        self.b_qkv = self.b_o = None
        if self.bias:
            self.b_qkv = torch.cat([w[n + ".bias"].float() for n in ("q_proj", "k_proj", "v_proj")]).contiguous()
            self.b_o = w["out_proj.bias"].float().contiguous()
        self.q_w = self.k_w = None
        if self.qk_norm_eps is not None:
            self.q_w = w["q_norm.weight"].float().contiguous()
            self.k_w = w["k_norm.weight"].float().contiguous()

    def cache_spec(self):
        return PagedKVSpec(self.G, self.hd, self.window)

    def forward(self, h, residual, ctx, cache):
        """``cache``: a :class:`~kappai_b200.cache.storage.KVLayerView`."""
        H, G, hd = self.H, self.G, self.hd
        view = ctx.paged[cache.group]
        qkv = linear(h, self.w_qkv, self.b_qkv)
        q = torch.empty((ctx.n_rows, H * hd), dtype=qkv.dtype, device=qkv.device)
        kv_out = cache.tensor if cache.writes else None
        if hasattr(self.position, "fused_rotary"):
            cos, sin, rot, inter = self.position.fused_rotary()
            K.qk_norm_rope_kv(qkv, self.q_w, self.k_w, self.qk_norm_eps or 0.0, cos, sin, rot, inter,
                              ctx.positions, view.slot_map, q, kv_out, view.page_size, H, G, hd)
        else:
            # a position encoding of its own: norm in place, let it change q and k, then scatter
            if self.q_w is not None:
                K.qk_norm_rope_kv(qkv, self.q_w, self.k_w, self.qk_norm_eps, None, None, 0, False, ctx.positions,
                                  None, None, None, view.page_size, H, G, hd)
            self.position.apply(qkv[:, :H * hd], qkv[:, H * hd:(H + G) * hd], ctx)
            K.qk_norm_rope_kv(qkv, None, None, 0.0, None, None, 0, False, ctx.positions, view.slot_map, q, kv_out,
                              view.page_size, H, G, hd)
        o = torch.empty_like(q)
        tiles = ctx.tables.get(self.step_tables_key)
        if self.split_ok and (tiles is None or q.dtype == torch.float32):
            # rows that each read a long cache (decode): split the keys over many CTAs.  The 32-bit path
            # takes this kernel for every row, whatever the length of its segment: its chunks lie at absolute
            # multiples of 256 keys and are summed in order, so a row's bits do not depend on how the step was cut.
            self._split(q, o, ctx, view, cache, ctx.n_rows)
        elif tiles is not None and K.attention_prefill_ok(q, hd):
            lead = tiles.n_short_rows
            if lead and self.split_ok:
                # decoded tokens beside prompt portions: the decoded rows lead the batch and go to the split
                # kernel (in a row tile each would walk its whole cache alone), the portions to the tiled one
                self._split(q, o, ctx, view, cache, lead)
                t0 = tiles.n_short_tiles
                K.attention_prefill(q, cache.tensor, view.block_table, ctx.cu_rows, ctx.seg_pos, tiles.tile_seg[t0:],
                                    tiles.tile_row0[t0:], o, self.scale, self.window, view.page_size, H, G, hd,
                                    tiles.big_tile_seg, tiles.big_tile_row0)
            else:
                # (with a lead that the split kernel cannot take, the big tiles leave it out: small tiles only)
                big = (None, None) if lead else (tiles.big_tile_seg, tiles.big_tile_row0)
                K.attention_prefill(q, cache.tensor, view.block_table, ctx.cu_rows, ctx.seg_pos, tiles.tile_seg,
                                    tiles.tile_row0, o, self.scale, self.window, view.page_size, H, G, hd, *big)
        else:
            K.attention_rows(q, cache.tensor, view.block_table, ctx.row_seg, ctx.positions, o, self.scale,
                             self.window, view.page_size, H, G, hd)
        linear(o, self.w_o, self.b_o, out=residual, accumulate=True)


    def _split(self, q, o, ctx, view, cache, n_rows):
        """Split-key attention for the first ``n_rows`` rows of the step."""
        H, G, hd = self.H, self.G, self.hd
        n_chunks = -(-ctx.max_context // K.SPLIT_CHUNK)
        need = K.attention_split_scratch(n_rows, H, hd, n_chunks)
        ws = self.env.shared.get("attn_scratch")
        if ws is None or ws.numel() < need:
            # A captured decode step keeps the address of the scratch it was captured with, so a buffer that
            # has been outgrown is retired, never freed: a replay of an older graph then still writes memory
            # that nobody else owns.  Growth doubles, so the retired buffers together are smaller than the live one.
            if ws is not None:
                self.env.shared.setdefault("attn_scratch_retired", []).append(ws)
            ws = torch.zeros(max(need, 2 * (ws.numel() if ws is not None else 0), 1 << 16), dtype=torch.float32,
                             device=q.device)
            self.env.shared["attn_scratch"] = ws
        K.attention_split(q[:n_rows], cache.tensor, view.block_table, ctx.row_seg[:n_rows], ctx.positions[:n_rows],
                          o[:n_rows], ws, n_chunks, self.scale, self.window, view.page_size, H, G, hd)


register_part("mixer", "attention", Attention)
