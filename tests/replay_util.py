"""Helpers of the trace-replay tests: build traces in the families the engine
must agree on, run ``bin/trace_run`` as a child process, and compare what it
wrote with the plain implementation."""
import json
import os
import random
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


class Trace:
    """Steps plus, for each, which (request, position) every written row is."""

    def __init__(self):
        self.steps = []          # dicts as trace_run reads them
        self.rows = []           # per step: list of (request, position)
        self.fed = {}            # request -> tokens fed so far

    def add(self, entries, end=()):
        """entries: list of (request, tokens, want indices)."""
        step = {"step": len(self.steps), "entries": [], "end": list(end)}
        rows = []
        for rid, toks, want in entries:
            base = self.fed.get(rid, 0)
            step["entries"].append({"id": rid, "tokens": [int(t) for t in toks], "want": [int(w) for w in want]})
            rows += [(rid, base + int(w)) for w in want]
            self.fed[rid] = base + len(toks)
        for rid in end:
            self.fed.pop(rid, None)
        self.steps.append(step)
        self.rows.append(rows)


def whole(trace, reqs):
    """Each request alone, whole, in one step; all positions wanted."""
    for rid, toks in reqs.items():
        trace.add([(rid, toks, range(len(toks)))], end=[rid])


def last_decoded(trace, reqs, n_last=32):
    """Most of it in one step, the last ``n_last`` tokens one by one."""
    for rid, toks in reqs.items():
        n0 = max(1, len(toks) - n_last)
        trace.add([(rid, toks[:n0], [n0 - 1])])
        for i in range(n0, len(toks)):
            trace.add([(rid, toks[i:i + 1], [0])], end=[rid] if i == len(toks) - 1 else [])
        if n0 == len(toks):
            trace.add([], end=[rid])


def portions(trace, reqs, sizes=(7, 2, 16, 3, 2, 5, 2, 31, 4, 2, 64, 2, 9)):
    """Portions of changing size, down to two tokens; all positions wanted."""
    for rid, toks in reqs.items():
        i, k = 0, 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            if len(toks) - i - n == 1:       # do not leave a lone token: the family is about portions
                n += 1
            k += 1
            last = i + n == len(toks)
            trace.add([(rid, toks[i:i + n], range(n))], end=[rid] if last else [])
            i += n


def mixed(trace, reqs, prompt_len, seed, max_live=4, page=64, max_tokens=None):
    """Up to ``max_live`` live requests; portions of some beside decoded tokens
    of others; a request may sit a step out; new ones start as others end.
    ``prompt_len[rid]`` tokens come in portions, the rest one by one.  If
    ``max_tokens`` is given a request only starts (or grows) while the live
    requests' page-rounded token counts stay within it."""
    rng = random.Random(seed)
    waiting = list(reqs)
    live = {}                                            # rid -> tokens fed
    rounded = lambda n: -(-n // page) * page
    while waiting or live:
        while waiting and len(live) < max_live:
            rid = waiting[0]
            if max_tokens is not None:
                held = sum(rounded(len(reqs[r])) for r in live)
                if held + rounded(len(reqs[rid])) > max_tokens:
                    break
            live[waiting.pop(0)] = 0
        entries, ended = [], []
        for rid in list(live):
            toks, fed = reqs[rid], live[rid]
            if rng.random() < 0.2 and len(live) > 1:
                continue                                 # sits this step out
            if fed < prompt_len[rid]:
                n = min(rng.choice([2, 2, 3, 5, 8, 13, 17, 30]), prompt_len[rid] - fed)
                if prompt_len[rid] - fed - n == 1:
                    n += 1
                want = sorted(set(rng.sample(range(n), min(n, 3))) | {n - 1})
            else:
                n, want = 1, [0]
            entries.append((rid, toks[fed:fed + n], want))
            live[rid] = fed + n
            if live[rid] == len(toks):
                ended.append(rid)
                del live[rid]
        if entries:
            trace.add(entries, end=ended)


def run_trace(model_dir, dtype, trace, out_dir, max_tokens, page_size=None, timeout=600, env=None):
    """Run trace_run over the trace, one step at a time (the next step is sent
    only after ``done <step>``).  Returns {step: array [wanted, vocab]}."""
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens)]
    if page_size is not None:
        cmd += ["--page-size", str(page_size)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                            env=env)
    try:
        for st in trace.steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            if line.strip() != f"done {st['step']}":
                err = proc.stderr.read()
                raise AssertionError(f"trace_run: expected 'done {st['step']}', got {line!r}\n{err[-3000:]}")
        proc.stdin.close()
        rc = proc.wait(timeout=timeout)
        if rc != 0:
            raise AssertionError(f"trace_run exited with {rc}\n{proc.stderr.read()[-3000:]}")
    finally:
        if proc.poll() is None:
            proc.kill()
    with open(os.path.join(model_dir, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    out = {}
    for st, rows in zip(trace.steps, trace.rows):
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if rows:
            a = np.fromfile(path, dtype="<f4")
            assert a.size == len(rows) * vocab, f"step {st['step']}: {a.size} floats for {len(rows)} rows"
            out[st["step"]] = a.reshape(len(rows), vocab)
        else:
            assert not os.path.exists(path), f"step {st['step']} wanted nothing but wrote a file"
    return out


def cache_stats(out_dir):
    with open(os.path.join(out_dir, "cache_stats.json")) as f:
        return json.load(f)


def rows_by_place(trace, outputs, first_step=0, last_step=None):
    """(request, position) -> the logits rows written for it in steps [first_step, last_step)."""
    out = {}
    for st, rows in zip(trace.steps, trace.rows):
        if rows and first_step <= st["step"] < (len(trace.steps) if last_step is None else last_step):
            for j, place in enumerate(rows):
                out.setdefault(place, []).append(outputs[st["step"]][j])
    return out


def compare(trace, outputs, expected, tol, what):
    """expected: request -> [T, vocab] logits of the plain implementation.
    Reports the first wrong (step, request, position)."""
    worst = 0.0
    for st, rows in zip(trace.steps, trace.rows):
        if not rows:
            continue
        got = outputs[st["step"]]
        for j, (rid, pos) in enumerate(rows):
            err = float(np.abs(got[j].astype(np.float64) - expected[rid][pos]).max())
            worst = max(worst, err)
            if not err <= tol:
                raise AssertionError(f"{what}: step {st['step']} request {rid!r} position {pos}: "
                                     f"max |logit error| {err:.3e} > {tol:.3e} "
                                     f"(entries of the step: {[(e['id'], len(e['tokens'])) for e in st['entries']]})")
    return worst
