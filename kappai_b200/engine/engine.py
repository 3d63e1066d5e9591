"""The engine: requests in, tokens out.

``Engine`` ties the step function (:class:`ModelRunner`), the scheduler and
the sampler into the loop ``schedule -> step -> sample -> update``; the
reference's loop is ``worker_main`` (src/server/openai.c:1545-1575) over
``context_decode_loop`` (src/context.c:1312-1457).  Tokens go in and come out
as ids: text is not part of the engine.
"""
from __future__ import annotations

import itertools
import logging
import sys
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence

import torch

from ..sampling.params import SamplingParams
from ..sampling.rng import resolve_seed
from ..sampling.sampler import sample
from ..ops import kernels as K
from .runner import EngineError, ModelRunner, StepEntry
from .scheduler import RUNNING, Request, ScheduledEntry, Scheduler


log = logging.getLogger("kappai_b200")       # --debug turns its DEBUG level on: one line a step


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
    kv_tokens: int = 0                 # tokens the page pools hold (0: max_batch * ctx_size, or what fits beside the weights)
    device: str = "cuda:0"
    look_ahead: bool = True            # launch the next decode step before the last one's tokens are read
    time_kernels: bool = False         # --time: device time by kernel class (steps run eagerly meanwhile)
    debug_forward: bool = False        # --debug-forward: per-layer statistics of the first step, top logits at every sample


@dataclass
class StepStats:
    n_steps: int = 0
    prompt_tokens: int = 0
    decode_tokens: int = 0
    prompt_seconds: float = 0.0
    decode_seconds: float = 0.0
    first_token_seconds: Optional[float] = None


@dataclass
class _Launched:
    """A step that runs (or has run) on the device and whose sampled tokens are on their way to the host."""

    plan: List[ScheduledEntry]
    got: List[Request]                         # the requests that sample in it, in the order of ``tokens``
    tokens: Optional[torch.Tensor]             # their new tokens on the device (int32)
    host: torch.Tensor                         # the pinned buffer the tokens and the status word are copied to
    done: torch.cuda.Event                     # recorded behind that copy


class Engine:
    """``step`` keeps the device busy while the host does its bookkeeping: once a step's sampled tokens
    are on their way to the host, and the next step can only be "every running request decodes one more
    token", that next step is launched at once, fed by the sampled tokens where they lie on the device; only
    then does the host wait for the first step's tokens, record them and return them.  The next call finds its
    step already running.  A request that ended meanwhile (end-of-sequence token, abort) had one row too many
    computed; the row is dropped, and rows of a batch do not depend on one another.  A step is launched ahead
    only if no request waits, every running request decodes, none reaches its length limits with the token
    under way, none has a repeat penalty (which reads the token history on the host), and pages for the next
    token are there without preempting anyone."""

    def __init__(self, args: EngineArgs, free_memory=None):
        from ..ops.kernels import MAX_STEP_ROWS
        from .runner import EngineError

        self.args = args
        if not (1 <= args.max_step_tokens <= MAX_STEP_ROWS):
            raise EngineError(f"max_step_tokens={args.max_step_tokens}: a step takes 1 to {MAX_STEP_ROWS} tokens")
        if args.max_batch < 1 or args.ctx_size < 0 or args.kv_tokens < 0:
            raise EngineError("max_batch must be positive; ctx_size and kv_tokens must not be negative")
        # the longest sequence is the model's own limit unless ctx_size asks for less (src/context.c:465-470);
        # the pools hold kv_tokens, or what max_batch requests of that length need, or what fits beside the weights
        self.runner = ModelRunner(args.model, dtype=args.dtype, max_tokens=args.kv_tokens, max_requests=args.max_batch,
                                  page_size=args.page_size, max_model_len=args.ctx_size or (1 << 62), device=args.device,
                                  max_step_tokens=args.max_step_tokens, free_memory=free_memory)
        self.scheduler = Scheduler(self.runner.cache, args.max_step_tokens, args.max_batch,
                                   self.runner.max_model_len, self.runner.spec.eos_token_id)
        self.requests: Dict[Hashable, Request] = {}
        self._ids = itertools.count()
        self.stats = StepStats()
        self._launched: Optional[_Launched] = None          # a step launched ahead by the last call of step()
        # two pinned buffers for sampled tokens: one is read while the step ahead fills the other
        # (one more element than tokens: the step's status word travels with them)
        self._token_staging = [torch.empty(max(args.max_batch, 1) + 1, dtype=torch.int32, pin_memory=True)
                               for _ in range(2)]
        self._staging_turn = 0
        self.n_launched_ahead = 0
        self.status = K.StatusGather(self.runner.device)
        self.timer: Optional[K.KernelTimer] = None
        if args.time_kernels:
            self.timer = K.KernelTimer()
            K.TIMER[0] = self.timer
        self._debug_steps = 0
        if args.debug_forward:
            self.runner.observer = self._observe_layer

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

    def abort(self, request_id: Hashable) -> None:
        """End a request now (``finish_reason`` "aborted"); what it holds is given back.  A row computed for it
        by a step that is already under way is dropped."""
        self.scheduler.abort(request_id)

    # -- debugging aids
    def _observe_layer(self, where: int, x: torch.Tensor) -> None:
        """--debug-forward: statistics of the residual behind every layer, for the first step only
        (the reference prints per-layer activation statistics for the first token, src/config.c:150)."""
        if self._debug_steps > 0:
            return
        spec = self.runner.spec
        name = "embedding" if where < 0 else f"layer {where:3d} ({spec.layers[spec.schedule[where].layer].mixer.kind})"
        v = x.float()
        print(f"[debug-forward] {name:<28} rows {v.shape[0]:5d}  min {v.min().item():+.6e}  max {v.max().item():+.6e}  "
              f"mean {v.mean().item():+.6e}  rms {v.pow(2).mean().sqrt().item():.6e}", file=sys.stderr)

    def _debug_logits(self, logits: torch.Tensor, got: List[Request]) -> None:
        """--debug-forward: the eight largest logits of every row that is sampled (src/context.c:1175-1211)."""
        top = torch.topk(logits.float(), min(8, logits.shape[1]), dim=1)
        for r, vals, idx in zip(got, top.values.tolist(), top.indices.tolist()):
            print(f"[debug-forward] request {r.id!r} top logits: " + " ".join(f"[{i}]={v:.4f}" for i, v in zip(idx, vals)),
                  file=sys.stderr)

    # -- one turn of the loop
    def _launch(self, plan: List[ScheduledEntry], device_tokens: Optional[torch.Tensor] = None,
                ahead: int = 0) -> _Launched:
        """Run the step for ``plan``, sample, and start the copy of the new tokens to the host; nothing
        waits.  With ``device_tokens`` every entry is one decoded token whose id lies on the device (the
        tokens sampled by the step before, which the host has not seen yet: ``ahead`` = 1)."""
        entries = []
        for e in plan:
            toks = [0] if device_tokens is not None else e.request.token_slice(e.start, e.n)
            entries.append(StepEntry(e.request.id, toks, [e.n - 1] if e.sample else []))
        logits = self.runner.step(entries, device_tokens=device_tokens)
        got = [e.request for e in plan if e.sample]
        if self.args.debug_forward:
            self._debug_steps += 1
            if got:
                self._debug_logits(logits, got)
        n = len(got)
        # the new tokens and, behind them, one word that says whether a kernel of the step gave up a wait
        buf = torch.empty(n + 1, dtype=torch.int32, device=self.runner.device)
        toks = None
        if got:
            # the token history only where a repeat penalty reads it
            recent = [r.tokens for r in got] if any(r.params.repeat_penalty != 1.0 for r in got) else None
            toks = sample(logits, [r.params for r in got], [r.seed for r in got],
                          [len(r.output) + ahead for r in got], recent, out=buf[:n])
        self.status.gather(buf[n:])
        host = self._token_staging[self._staging_turn]
        self._staging_turn ^= 1
        host[:n + 1].copy_(buf, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return _Launched(plan, got, toks, host, done)

    def _launch_ahead(self, cur: _Launched) -> Optional[_Launched]:
        """The step after ``cur``, if it can only be one more token for every request of ``cur``."""
        sch = self.scheduler
        if (not self.args.look_ahead or sch.waiting or not cur.got or len(cur.got) != len(cur.plan)
                or len(cur.plan) != len(sch.running)):
            return None
        for r in cur.got:
            n_pred = r.params.n_predict
            if (r.state != RUNNING or r.params.repeat_penalty != 1.0
                    or (n_pred >= 0 and len(r.output) + 1 >= n_pred)
                    or r.n_tokens + 1 >= self.runner.max_model_len):
                return None
        for r in cur.got:
            if not self.runner.cache.try_extend(r.id, r.n_tokens + 1):
                return None                 # (pages taken for the others stay theirs: they need them anyway)
        plan = [ScheduledEntry(r, r.n_tokens, 1, True) for r in cur.got]
        self.n_launched_ahead += 1
        return self._launch(plan, device_tokens=cur.tokens, ahead=1)

    def step(self) -> List[Request]:
        """Schedule, run and sample one step; returns the requests that got a new token."""
        t0 = time.perf_counter()
        cur, self._launched = self._launched, None
        if cur is not None and not any(e.request.state == RUNNING for e in cur.plan):
            cur.done.synchronize()                                   # everyone in it has ended meanwhile
            cur = None
        if cur is None:
            plan = self.scheduler.schedule()
            if not plan:
                return []
            cur = self._launch(plan)
        ahead = self._launch_ahead(cur)
        cur.done.synchronize()                                       # the step's one device-to-host read
        new = cur.host[:len(cur.got) + 1].tolist()
        if new.pop():
            self._compute_failed(cur, ahead)
        plan = [e for e in cur.plan if e.request.state == RUNNING]   # without those that ended meanwhile
        sampled = {r.id: t for r, t in zip(cur.got, new)}
        n_prompt = sum(e.n for e in plan if e.n > 1 or not e.request.output)
        n_decode = sum(1 for e in plan if e.n == 1 and e.request.output and e.sample)
        self.scheduler.update(plan, sampled)
        self._launched = ahead
        got = [e.request for e in plan if e.sample]
        dt = time.perf_counter() - t0
        if log.isEnabledFor(logging.DEBUG):
            log.debug("step %d: %s | %.3f ms | running %d waiting %d | pages free %s | preemptions %d%s",
                      self.stats.n_steps, " ".join(f"{e.request.id!r}:{e.start}+{e.n}" for e in plan), dt * 1e3,
                      len(self.scheduler.running), len(self.scheduler.waiting),
                      "/".join(str(p.n_free) for p in self.runner.cache.pools.values()) or "-",
                      self.scheduler.n_preemptions,
                      "".join(f" | {r.id!r} finished: {r.finish_reason}" for r in got if r.finish_reason))
        st = self.stats
        st.n_steps += 1
        if n_prompt >= n_decode:
            st.prompt_seconds += dt
        else:
            st.decode_seconds += dt
        st.prompt_tokens += n_prompt
        st.decode_tokens += len(got)
        return got

    def _compute_failed(self, cur: _Launched, ahead: Optional[_Launched]) -> None:
        """A kernel of the step gave up a bounded wait (src/context.c:1580-1592: a compute failure ends the
        session): what the step computed cannot be trusted, nor what a step launched ahead made of it.  Their
        requests end with ``compute_failed``, pages and slots return, the status words are cleared, and the
        caller is told.  Requests that were not in the step go on."""
        if ahead is not None:
            ahead.done.synchronize()
        what = self.status.clear()
        reqs = {id(e.request): e.request for l in (cur, ahead) if l is not None for e in l.plan}
        self.scheduler.fail(list(reqs.values()))
        self.stats.n_steps += 1
        raise EngineError("a kernel's bounded wait gave up (" + ", ".join(sorted(what)) + "): the step's requests "
                          + ", ".join(repr(r.id) for r in reqs.values()) + " ended with compute_failed")

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
        if self.timer is not None and K.TIMER[0] is self.timer:
            K.TIMER[0] = None
        if self._launched is not None:
            self._launched.done.synchronize()
            self._launched = None
        self.runner = None
        self.scheduler = None
