"""The step function: one batch of (request, its next tokens) from the cache.

``ModelRunner`` owns the model, the device cache and the cache manager, and
runs steps.  A step takes, for each request in it, that request's next tokens
(a portion of a prompt, cut anywhere, or one decoded token) and the places
among them whose logits are wanted; it runs only those tokens, as one batch,
reading what earlier steps left in the cache, and returns the logits at the
wanted places.  The reference's step function has the same contract
(src/recipe/exec.c:704-758: embed rows, run layers, gather the rows that need
logits, final norm, head).

Everything above (scheduler, sampling, trace replay, the entry points) drives
this one function; there is no second forward pass.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import CacheManager, OutOfPages
from ..cache.spec import PagedKVSpec, StateSpec
from ..cache.storage import CacheStorage
from ..config.registry import load_config
from ..parts.base import BuildEnv
from ..weights.loader import load_weights
from .batch import Segment, StepContext, lay_out_step, upload_step
from ..ops import kernels as K
from ..ops.kernels import MAX_STEP_ROWS
from .graphs import DecodeGraphs
from .memory import CacheMemoryError, GroupNeed, plan_cache
from .model import Model

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class EngineError(RuntimeError):
    pass


@dataclass
class StepEntry:
    req: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise EngineError(f"kappai_b200 runs on a CUDA device only, not '{device}'")
    if not torch.cuda.is_available():
        raise EngineError("no CUDA device is available; kappai_b200 has no CPU path")
    return device


class ModelRunner:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", max_tokens: int = 4096,
                 max_requests: int = 4, page_size: int = 64, max_model_len: Optional[int] = None,
                 device="cuda:0", cuda_graphs: bool = True, max_step_tokens: Optional[int] = None,
                 free_memory=None):
        """``max_tokens``: how many tokens the live requests may hold together,
        each request's count rounded up to a whole page; the page pools are
        made for exactly this many, or the runner refuses to start if the device
        has no room for them.  0: room for ``max_requests`` requests of
        ``max_model_len`` tokens, or as much of that as fits beside the weights.
        ``max_requests``: state slots.  ``cuda_graphs``: replay decode steps
        from captured CUDA graphs.  ``max_step_tokens``: the most tokens a
        request gets in one step, if the caller keeps such a limit: pools of
        windowed page groups are then made no larger than the windows need.
        ``free_memory``: a function that returns the device's free bytes (for
        tests; by default the device is asked)."""
        if dtype not in DTYPES:
            raise EngineError(f"dtype '{dtype}': expected bfloat16 or float32")
        self.device = require_cuda(device)
        self.dtype = DTYPES[dtype]
        self.arch, self.config = load_config(model_dir)
        self.spec = self.arch.build_spec(self.config)
        if page_size < 1:
            raise EngineError("page_size must be positive")
        if max_tokens < 0 or max_requests < 1:
            raise EngineError("max_tokens must not be negative and max_requests must be positive")
        self.page_size = page_size
        limit = max_model_len or (-(-max_tokens // page_size) * page_size if max_tokens else self.spec.max_positions)
        self.max_model_len = min(self.spec.max_positions, limit)
        torch.cuda.set_device(self.device)
        env = BuildEnv(self.device, self.dtype, self.max_model_len)
        self.model = Model(self.spec, env)
        load_weights(self.model, model_dir)
        specs = self.model.cache_specs()
        borrowing = self.model.cache_borrowing()
        elt = torch.empty((), dtype=self.dtype).element_size()
        needs: Dict[Hashable, GroupNeed] = {}
        state_bytes = 0
        for s in specs:
            if isinstance(s, PagedKVSpec):
                g = needs.setdefault(s.group_key, GroupNeed(s.group_key, 0, s.window))
                g.bytes_per_token += 2 * s.num_kv_heads * s.head_dim * elt
            elif isinstance(s, StateSpec):
                n = 1
                for d in s.shape:
                    n *= d
                state_bytes += n * torch.empty((), dtype=getattr(torch, s.dtype)).element_size()
        free = free_memory() if free_memory is not None else torch.cuda.mem_get_info(self.device)[0]
        try:
            plan = plan_cache(list(needs.values()), state_bytes, max_requests, page_size, self.max_model_len,
                              max_tokens, free, max_step_tokens)
        except CacheMemoryError as e:
            raise EngineError(str(e)) from None
        self.cache_plan = plan
        group_keys = list(needs)
        self.storage = CacheStorage(specs, borrowing, plan.pages, page_size, max_requests, self.dtype, self.device)
        self.cache = CacheManager({gk: (plan.pages[gk], page_size, self.storage.groups[gk].window)
                                   for gk in group_keys}, max_requests)
        self.group_page_size = {gk: page_size for gk in group_keys}
        self.vocab_size = self.spec.vocab_size
        self.last_h2d_bytes = 0
        self.observer = None               # called with the residual behind every layer of a step (debugging): see Model.forward
        self.graphs: Optional[DecodeGraphs] = DecodeGraphs(self) if cuda_graphs else None

    # -- requests
    def is_live(self, req: Hashable) -> bool:
        return req in self.cache.requests

    def length(self, req: Hashable) -> int:
        return self.cache.requests[req].length

    def end(self, req: Hashable) -> None:
        """The request is finished: its pages and its slot are given back."""
        self.cache.free(req)

    def can_run(self, req: Hashable, n_new: int) -> bool:
        """Would pages (and, for a new request, a slot) be there for ``n_new`` more tokens?"""
        if req in self.cache.requests:
            return self.cache.can_extend(req, self.cache.requests[req].length + n_new)
        if not self.cache.can_admit():
            return False
        return all(-(-n_new // p.page_size) <= p.n_free for p in self.cache.pools.values())

    def check_status(self) -> None:
        """Wait for the device and raise if a kernel gave up a bounded wait since the last check (its output
        is then not to be trusted).  The status words are cleared."""
        bad = sorted(k for k, v in K.read_status().items() if v)
        if bad:
            raise EngineError("a kernel's bounded wait gave up (" + ", ".join(bad) + "): the results of the "
                              "steps since the last check are not valid")

    # -- the step
    def _reserve(self, entries: Sequence[StepEntry]) -> List[Tuple[Hashable, int, int]]:
        """Admit new requests and take pages for every entry's new tokens.
        Returns (request, length before, length after) per entry.  Nothing is
        kept of a new request if any entry cannot be served."""
        n_rows = sum(len(e.tokens) for e in entries)
        if n_rows > MAX_STEP_ROWS:
            raise EngineError(f"a step of {n_rows} tokens exceeds the kernels' limit of {MAX_STEP_ROWS} rows a step")
        admitted = []
        try:
            plan = []
            for e in entries:
                if len(e.tokens) < 1:
                    raise EngineError(f"request {e.req!r}: no tokens in this step")
                if e.req not in self.cache.requests:
                    self.cache.admit(e.req)
                    admitted.append(e.req)
                rc = self.cache.requests[e.req]
                new_len = rc.length + len(e.tokens)
                if new_len > self.max_model_len:
                    raise EngineError(f"request {e.req!r}: {new_len} tokens exceed the limit of "
                                      f"{self.max_model_len} positions")
                self.cache.extend(e.req, new_len)
                plan.append((e.req, rc.length, new_len))
            if len({p[0] for p in plan}) != len(plan):
                raise EngineError("a request appears twice in one step")
            return plan
        except Exception:
            for r in admitted:
                self.cache.free(r)
            # pages taken for requests that were already live stay with them: they
            # cover positions the request will need anyway and are freed with it
            raise

    def _lay_out(self, entries: Sequence[StepEntry], capturable: bool):
        """Reserve cache for the entries and lay the step's tables out on the host."""
        plan = self._reserve(entries)
        segs = []
        for e, (req, old_len, new_len) in zip(entries, plan):
            rc = self.cache.requests[req]
            segs.append(Segment(
                req=req, tokens=e.tokens, pos_start=old_len, want=e.want, slot=rc.slot,
                block_tables={gk: self.cache.block_table(req, gk) for gk in self.group_page_size},
                token_slots={gk: self.cache.token_slots(req, gk, old_len, len(e.tokens))
                             for gk in self.group_page_size}))
        g = self.graphs if capturable else None
        host = lay_out_step(segs, self.group_page_size, self.vocab_size, self.max_model_len, self.model.table_builders,
                            round_blocks=g.round_blocks if g else None,
                            round_context=(lambda t: min(self.max_model_len, g.round_context(t))) if g else None)
        return host, [(req, new_len) for req, _, new_len in plan]

    def prepare(self, entries: Sequence[StepEntry]) -> Tuple[StepContext, List[Tuple[Hashable, int]]]:
        """Reserve cache for the entries and build the step's tables."""
        host, after = self._lay_out(entries, False)
        return upload_step(host, self.device), after

    def run(self, ctx: StepContext) -> Optional[torch.Tensor]:
        return self.model.forward(ctx, self.storage.views, self.observer)

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None
             ) -> Optional[torch.Tensor]:
        """Run one step; float32 logits [wanted, vocab] on the device, in the
        order of the entries and of their ``want`` (None if nothing is wanted).
        With ``device_tokens`` (int32, one per row, on the device) the token ids
        of the entries are placeholders and those are run instead, so sampled
        tokens need not visit the host between steps.  The returned tensor may
        be reused by the next step: read it before."""
        if (self.graphs is not None and self.model.graph_safe and self.observer is None and K.TIMER[0] is None
                and DecodeGraphs.eligible(entries) and self.graphs.wants(entries)):
            for e in entries:
                if not (0 <= int(e.tokens[0]) < self.vocab_size):
                    raise EngineError(f"request {e.req!r}: token id {e.tokens[0]} outside the vocabulary")
            plan = self._reserve(entries)
            logits = self.graphs.step(entries, device_tokens)
            for req, _, new_len in plan:
                self.cache.advance(req, new_len)
            return logits
        # (a decode step that is not captured yet runs as it is; other shapes may be captured as they are laid out)
        capturable = (self.graphs is not None and self.model.graph_safe and self.observer is None
                      and K.TIMER[0] is None and not DecodeGraphs.eligible(entries))
        host, after = self._lay_out(entries, capturable)
        if capturable and self.graphs.wants_step(host):
            # a shape that has come before: from its captured graph (see DecodeGraphs.run_step)
            logits = self.graphs.run_step(host, device_tokens)
        else:
            ctx = upload_step(host, self.device)
            if device_tokens is not None:
                ctx.token_ids.copy_(device_tokens)
            self.last_h2d_bytes = ctx.h2d_bytes
            logits = self.run(ctx)
        for req, new_len in after:
            self.cache.advance(req, new_len)
        return logits
