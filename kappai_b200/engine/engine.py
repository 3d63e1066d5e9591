"""The engine: requests in, tokens out.

``Engine`` ties the step function (:class:`ModelRunner`), the scheduler and
the sampler into the loop ``schedule -> step -> sample -> update``; the
reference's loop is ``worker_main`` (src/server/openai.c:1545-1575) over
``context_decode_loop`` (src/context.c:1312-1457).  Tokens go in and come out
as ids: text is not part of the engine.
"""
from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence

import torch

from ..sampling.params import SamplingParams
from ..sampling.rng import resolve_seed
from ..sampling.sampler import sample
from .runner import ModelRunner, StepEntry
from .scheduler import Request, ScheduledEntry, Scheduler


@dataclass
class EngineArgs:
    """Engine options.  Names follow the reference's flags where it has them
    (src/config.c:48-61,84-118): ``model`` (-m), ``ctx_size`` (-c, 0 = from the
    model)."""

    model: str = ""
    dtype: str = "bfloat16"            # "float32": the whole model in true 32-bit
    ctx_size: int = 0                  # longest sequence (0: the model's max_position_embeddings)
    max_batch: int = 64                # requests that run together (state slots)
    max_step_tokens: int = 2048        # token budget of one step
    page_size: int = 64
    kv_tokens: int = 0                 # tokens the page pools hold (0: max_batch * ctx_size, capped by memory)
    device: str = "cuda:0"


@dataclass
class StepStats:
    n_steps: int = 0
    prompt_tokens: int = 0
    decode_tokens: int = 0
    prompt_seconds: float = 0.0
    decode_seconds: float = 0.0
    first_token_seconds: Optional[float] = None


class Engine:
    def __init__(self, args: EngineArgs):
        from ..config.registry import load_config

        self.args = args
        _, cfg = load_config(args.model)
        arch_ctx = getattr(cfg, "max_position_embeddings", None) or 4096
        ctx_size = min(args.ctx_size or arch_ctx, arch_ctx)         # src/context.c:465-470
        kv_tokens = args.kv_tokens or min(args.max_batch * ctx_size, 1 << 22)
        self.runner = ModelRunner(args.model, dtype=args.dtype, max_tokens=kv_tokens, max_requests=args.max_batch,
                                  page_size=args.page_size, max_model_len=ctx_size, device=args.device)
        self.scheduler = Scheduler(self.runner.cache, args.max_step_tokens, args.max_batch,
                                   self.runner.max_model_len, self.runner.spec.eos_token_id)
        self.requests: Dict[Hashable, Request] = {}
        self._ids = itertools.count()
        self.stats = StepStats()

    @property
    def vocab_size(self) -> int:
        return self.runner.vocab_size

    # -- requests
    def add_request(self, tokens: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None) -> Hashable:
        params = params or SamplingParams()
        params.validate(self.vocab_size)
        rid = request_id if request_id is not None else next(self._ids)
        if rid in self.requests:
            raise ValueError(f"request id {rid!r} is already in use")
        for t in tokens:
            if not (0 <= int(t) < self.vocab_size):
                raise ValueError(f"token id {t} outside the vocabulary of {self.vocab_size}")   # src/context.c:866-867
        req = Request(rid, [int(t) for t in tokens], params, seed=resolve_seed(params.seed))
        self.scheduler.add(req)
        self.requests[rid] = req
        return rid

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    # -- one turn of the loop
    def step(self) -> List[Request]:
        """Schedule, run and sample one step; returns the requests that got a new token."""
        t0 = time.perf_counter()
        plan = self.scheduler.schedule()
        if not plan:
            return []
        entries = []
        for e in plan:
            toks = e.request.token_slice(e.start, e.n)
            entries.append(StepEntry(e.request.id, toks, [e.n - 1] if e.sample else []))
        logits = self.runner.step(entries)
        sampled: Dict[Hashable, int] = {}
        got = [e.request for e in plan if e.sample]
        if got:
            # the token history only where a repeat penalty reads it
            recent = [r.tokens for r in got] if any(r.params.repeat_penalty != 1.0 for r in got) else None
            toks = sample(logits, [r.params for r in got], [r.seed for r in got], [len(r.output) for r in got],
                          recent)
            for r, t in zip(got, toks.tolist()):                    # the step's one device-to-host read
                sampled[r.id] = t
        else:
            torch.cuda.current_stream().synchronize()
        self.scheduler.update(plan, sampled)
        dt = time.perf_counter() - t0
        st = self.stats
        st.n_steps += 1
        n_prompt = sum(e.n for e in plan if e.n > 1 or not e.request.output)
        n_decode = sum(1 for e in plan if e.n == 1 and e.request.output and e.sample)
        if n_prompt >= n_decode:
            st.prompt_seconds += dt
        else:
            st.decode_seconds += dt
        st.prompt_tokens += n_prompt
        st.decode_tokens += len(got)
        return got

    # -- whole generations
    def generate(self, prompts: Sequence[Sequence[int]], params=None,
                 on_token: Optional[Callable[[Hashable, int], None]] = None) -> List[List[int]]:
        """Generate for every prompt (lists of token ids); returns the new token
        ids of each, in the order of ``prompts``.  ``params`` is one
        :class:`SamplingParams` for all or one per prompt."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while self.has_work():
            for r in self.step():
                if on_token is not None:
                    on_token(r.id, r.output[-1])
        return [self.requests[i].output for i in ids]

    def finish_reason(self, request_id: Hashable) -> Optional[str]:
        return self.requests[request_id].finish_reason

    def shutdown(self) -> None:
        self.runner = None
        self.scheduler = None
