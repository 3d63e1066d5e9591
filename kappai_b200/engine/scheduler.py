"""The scheduler: which requests run which tokens in the next step.

The reference's scheduler (src/server/openai.c:1511-1575) admits jobs from a
FIFO queue while slots are free, runs one prefill chunk per prefilling task
per loop turn and one decode batch over all decoding tasks, and never shares a
launch between the two.  Each of its slots owns a full-context KV region, so
pages cannot run out.  Here one step holds decode tokens and prompt portions
together, under a token budget, and pages are a shared pool:

* every step first gives each decoding request its one token, then fills the
  rest of the budget with prompt portions: running prefills first, then new
  requests from the FIFO queue while a state slot and pages are free and
  fewer than ``max_running`` requests run;
* a portion is cut wherever the budget ends (down to one token);
* logits are wanted only where a request's known tokens end (its next token
  is sampled there);
* when pages run out for a running request, the most recently admitted
  running request is preempted: its pages and slot are given back and it goes
  to the front of the queue with all its tokens so far, to be computed again
  (state of fixed size cannot be rolled back, so recomputing is the only exact
  way; the reference notes the same for rewinds, src/context.c:752-761).  A
  request that cannot get its pages although it runs alone is finished with
  ``out_of_memory``.

The scheduler takes pages and slots from the :class:`CacheManager` itself, so
its decisions can be tested with no device.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
FINISH_EOS, FINISH_LENGTH, FINISH_CONTEXT, FINISH_OOM, FINISH_ABORT, FINISH_COMPUTE = (
    "eos", "length", "context_full", "out_of_memory", "aborted", "compute_failed")


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    seed: int = 1                               # resolved seed (never 0)
    output: List[int] = field(default_factory=list)
    state: str = WAITING
    n_computed: int = 0                         # tokens whose keys/state are in the cache
    n_preempted: int = 0
    finish_reason: Optional[str] = None
    admit_order: int = -1

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def n_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    def token_slice(self, start: int, n: int) -> List[int]:
        """``tokens[start:start + n]`` without joining the two lists."""
        lp = len(self.prompt)
        if start >= lp:
            return self.output[start - lp:start - lp + n]
        if start + n <= lp:
            return self.prompt[start:start + n]
        return self.prompt[start:] + self.output[:start + n - lp]


@dataclass
class ScheduledEntry:
    request: Request
    start: int              # index of the first token of the portion in request.tokens
    n: int                  # tokens in the portion
    sample: bool            # the portion ends at the request's last known token


class Scheduler:
    def __init__(self, cache: CacheManager, max_step_tokens: int, max_running: int, max_model_len: int,
                 eos_token_id: Optional[int] = None):
        if max_step_tokens < 1 or max_running < 1:
            raise ValueError("max_step_tokens and max_running must be positive")
        self.cache = cache
        self.max_step_tokens, self.max_running = max_step_tokens, max_running
        self.max_model_len, self.eos_token_id = max_model_len, eos_token_id
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # in admission order
        self.finished: List[Request] = []
        self._admitted = 0
        self.n_preemptions = 0

    # -- requests
    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError("a request needs at least one prompt token")
        if len(req.prompt) >= self.max_model_len:
            raise ValueError(f"prompt of {len(req.prompt)} tokens leaves no room under the limit of "
                             f"{self.max_model_len} positions")
        req.state = WAITING
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def abort(self, req_id: Hashable) -> None:
        for r in list(self.running):
            if r.id == req_id:
                self._finish(r, FINISH_ABORT)
                return
        for r in list(self.waiting):
            if r.id == req_id:
                self.waiting.remove(r)
                r.state, r.finish_reason = FINISHED, FINISH_ABORT
                self.finished.append(r)
                return

    def fail(self, requests, reason: str = FINISH_COMPUTE) -> None:
        """A step's kernels failed: its requests end with ``reason`` and what they hold is given back (the
        reference ends a session whose compute failed, src/context.c:1580-1592,1676-1680)."""
        for r in requests:
            if r.state != FINISHED:
                if r in self.waiting:
                    self.waiting.remove(r)
                self._finish(r, reason)

    # -- one step's plan
    def schedule(self) -> List[ScheduledEntry]:
        budget = self.max_step_tokens
        entries: List[ScheduledEntry] = []
        preempted = False
        # decodes first (one token each), then running prefills, both in admission order
        order = [r for r in self.running if r.n_tokens - r.n_computed == 1] + \
                [r for r in self.running if r.n_tokens - r.n_computed > 1]
        for r in order:
            if r.state != RUNNING or budget == 0:
                continue
            n = min(r.n_tokens - r.n_computed, budget)
            while not self.cache.try_extend(r.id, r.n_computed + n):
                victim = self._victim(exclude=[e.request for e in entries])
                if victim is None or victim is r:
                    if len(self.running) == 1:
                        # alone and still no room: this request can never be served
                        self._finish(r, FINISH_OOM)
                    else:
                        self._preempt(r)
                        preempted = True
                    break
                self._preempt(victim)
                preempted = True
            if r.state != RUNNING:
                continue
            entries.append(ScheduledEntry(r, r.n_computed, n, r.n_computed + n == r.n_tokens))
            budget -= n
        # admission (not in a step that had to preempt: the freed pages are for those who run)
        while (self.waiting and budget > 0 and not preempted and len(self.running) < self.max_running
               and self.cache.can_admit()):
            r = self.waiting[0]
            n = min(r.n_tokens, budget)
            if not all(-(-n // p.page_size) <= p.n_free for p in self.cache.pools.values()):
                if not self.running and not entries:
                    # nothing runs, every page is free, and the first portion still does not fit
                    self.waiting.popleft()
                    r.state, r.finish_reason = FINISHED, FINISH_OOM
                    self.finished.append(r)
                    continue
                break
            self.waiting.popleft()
            self.cache.admit(r.id)
            self.cache.extend(r.id, n)
            r.state, r.n_computed = RUNNING, 0
            r.admit_order = self._admitted
            self._admitted += 1
            self.running.append(r)
            entries.append(ScheduledEntry(r, 0, n, n == r.n_tokens))
            budget -= n
        return entries

    def _victim(self, exclude) -> Optional[Request]:
        """The most recently admitted running request not already in this step's plan."""
        ex = {id(x) for x in exclude}
        cands = [r for r in self.running if id(r) not in ex]
        return max(cands, key=lambda r: r.admit_order) if cands else None

    def _preempt(self, r: Request) -> None:
        self.cache.free(r.id)
        self.running.remove(r)
        r.state, r.n_computed = WAITING, 0
        r.n_preempted += 1
        self.n_preemptions += 1
        self.waiting.appendleft(r)

    def _finish(self, r: Request, reason: str) -> None:
        if r.id in self.cache.requests:
            self.cache.free(r.id)
        if r in self.running:
            self.running.remove(r)
        r.state, r.finish_reason = FINISHED, reason
        self.finished.append(r)

    # -- after the step ran
    def update(self, entries: List[ScheduledEntry], sampled: Dict[Hashable, int]) -> List[Request]:
        """Record what the step computed; ``sampled`` maps request id -> the new
        token of every entry with ``sample``.  Returns the requests that finished."""
        done = []
        for e in entries:
            r = e.request
            r.n_computed = e.start + e.n
            if self.cache.requests[r.id].length < r.n_computed:       # (a step function may have done it)
                self.cache.advance(r.id, r.n_computed)
            if not e.sample:
                continue
            tok = int(sampled[r.id])
            r.output.append(tok)
            n_pred = r.params.n_predict
            if self.eos_token_id is not None and tok == self.eos_token_id:
                reason = FINISH_EOS                               # src/context.c:1399
            elif n_pred >= 0 and len(r.output) >= n_pred:
                reason = FINISH_LENGTH                            # src/context.c:1332
            elif r.n_tokens >= self.max_model_len:
                reason = FINISH_CONTEXT                           # src/context.c:1444-1448
            else:
                continue
            self._finish(r, reason)
            done.append(r)
        return done
