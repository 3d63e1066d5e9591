#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the LFM2-1.2B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--workload long|many]

One "step" is one decode step of the whole batch.  The default run has the
layer sizes of the LFM2-1.2B configuration with random weights (seed 2), a
batch of 8 requests, prompts of 2,048 tokens and a context limit of 4,096:
every request decodes from 2,048 to 4,096 tokens (2,048 steps), and CUDA events
mark windows of exactly K steps at the start, the middle and the end of that
run.  It prints one JSON line:

* ``value``: decoded tokens a second over the K steps in the middle of the run
  (context about 3,072; a step's time grows linearly with the context, so this
  is also the mean over 2,048 -> 4,096, which ``points`` gives beside it),
  timed on the device (sampled tokens stay on the device between steps);
* ``e2e``: the same through the Python entry point (``Engine.step``): host
  token ids in, host token ids out, every step;
* ``prefill``: one 2,048-token prompt in one step, on the device alone and
  from the building of the step's tables to the logits, with the fraction of
  the bf16 matrix peak;
* ``roofline``: bytes a decode step has to read (every weight once, the cache
  of the live requests) over its time, against the measured copy bandwidth;
* ``points``: the same run at batch 1 and 64, and for every batch the two
  ends of the run and its mean (tokens a second, milliseconds a step, bytes a
  step, fraction of the copy bandwidth).

``--workload long`` (LFM2-2.6B shape, 16 requests with prompts of 1k to 30k
tokens, portions of 2,048, context 32,768) and ``--workload many`` (LFM2-350M
shape, 256 requests at once, prompts of 16 to 512 tokens, 128 sampled tokens
each at temperature 0.8) run whole generations through ``Engine`` and print a
line of their own: tokens a second, steps, preemptions, mean step time.

Only one GPU is used; ``--gpus N`` with N > 1 prints a line that says so and
exits with 2.
"""
import argparse
import hashlib
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LFM2_1P2B = dict(
    architectures=["Lfm2ForCausalLM"], vocab_size=65536, hidden_size=2048, num_hidden_layers=16,
    num_attention_heads=32, num_key_value_heads=8,
    layer_types=["conv", "conv", "full_attention", "conv", "conv", "full_attention", "conv", "conv",
                 "full_attention", "conv", "full_attention", "conv", "full_attention", "conv",
                 "full_attention", "conv"],
    max_position_embeddings=128000, norm_eps=1e-5, conv_L_cache=3, conv_bias=False,
    block_ff_dim=8192, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256,
    rope_theta=1000000.0, tie_embedding=True)
LFM2_2P6B = dict(LFM2_1P2B, num_hidden_layers=30, block_ff_dim=10752,
                 layer_types=["full_attention" if i in (2, 6, 10, 14, 18, 21, 24, 27) else "conv" for i in range(30)])
LFM2_350M = dict(LFM2_1P2B, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, block_ff_dim=6656)
SEED = 2
PROMPT_LEN = 2048
CONTEXT = 4096

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(d.get(k), (int, float)) and d[k] > 0:
                    out[k] = float(d[k])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.t.join(timeout=2)
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            if len(s) < 6:
                continue
            try:
                mhz.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for n, v in zip(names, s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def model_folder(cfg, seed, n_layers):
    """A model folder with random weights in the temp dir, made once per configuration."""
    from kappai_b200.weights import write_random_model

    c = dict(cfg)
    if n_layers < cfg["num_hidden_layers"]:
        c["num_hidden_layers"] = n_layers
        c["layer_types"] = cfg["layer_types"][:n_layers]
    key = hashlib.sha256(json.dumps([c, seed], sort_keys=True).encode()).hexdigest()[:12]
    d = os.path.join(tempfile.gettempdir(), f"kappai_b200_bench_{os.getuid()}_{key}")
    if not (os.path.isfile(os.path.join(d, "model.safetensors")) and os.path.isfile(os.path.join(d, ".complete"))):
        t0 = time.time()
        print(f"[bench] writing random weights to {d} ...", file=sys.stderr, flush=True)
        write_random_model(c, d, seed)
        with open(os.path.join(d, ".complete"), "w") as f:
            f.write("ok")
        print(f"[bench] done in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return d, c


def weight_bytes(runner):
    """Bytes of every weight a decode step reads once (a tied table counts once;
    an untied embedding table is only gathered from, so it is left out)."""
    m = runner.model
    seen, total = set(), 0
    for part, _local, _ws in m._table.values():
        for v in vars(part).values():
            if hasattr(v, "data_ptr") and hasattr(v, "numel") and v.data_ptr() not in seen:
                seen.add(v.data_ptr())
                total += v.numel() * v.element_size()
    if not getattr(m.head, "tied", False):
        total -= m.embedding.weight.numel() * m.embedding.weight.element_size()
    return total


def matrix_params_per_token(runner):
    """Weight elements every token is multiplied with (all matrices of the layers)."""
    n = 0
    for b in runner.model.blocks:
        for part in (b.mixer, b.ffn):
            if part is None:
                continue
            for v in vars(part).values():
                if hasattr(v, "dim") and v.dim() == 2 and v.shape[0] > 1 and v.shape[1] > 16:
                    n += v.numel()
    return n


def attention_flops(runner, T):
    f = 0
    for b in runner.model.blocks:
        mx = b.mixer
        if hasattr(mx, "H") and hasattr(mx, "hd"):
            f += 2 * mx.hd * mx.H * T * (T + 1)          # QK^T and PV over the causal half
    return f


def cache_bytes_per_step(runner, batch, context):
    """Keys and values of the live requests (read once) plus their fixed-size state (read and written)."""
    from kappai_b200.cache.storage import StateView

    kv = sum(runner.storage.bytes_per_token(g) for g in runner.storage.pools) * context * batch
    st = 0
    for v in runner.storage.views:
        if isinstance(v, StateView) and v.writes:
            st += 2 * v.tensor[0].numel() * v.tensor.element_size() * batch
    return kv + st


def run_decode(runner, batch, prompt_len, context, steps, warmup, rng):
    """Prefill ``batch`` requests of ``prompt_len`` tokens, then decode every one of them up to ``context``
    tokens, on the device alone.  CUDA events mark three windows of exactly ``steps`` steps (after the warm-up,
    in the middle, at the end) and the whole run after the warm-up.  Returns a dict of windows
    name -> (ms a step, context at the window's middle) and the kernel launchers called in the middle window."""
    import torch
    from kappai_b200 import StepEntry
    from kappai_b200.ops import kernels as K
    from kappai_b200.sampling.sampler import argmax

    V = runner.vocab_size
    ids = [f"d{batch}_{i}" for i in range(batch)]
    tok = None
    for i, rid in enumerate(ids):                      # prefill one by one (untimed)
        logits = runner.step([StepEntry(rid, rng.integers(0, V, prompt_len).tolist(), [prompt_len - 1])])
        t = argmax(logits)
        tok = t if tok is None else torch.cat([tok, t])
    entries = [StepEntry(rid, [0], [0]) for rid in ids]
    n_steps = context - prompt_len                     # the step that makes a request context tokens long is the last
    if steps + warmup > n_steps:
        raise SystemExit(f"bench.py: --steps + --warmup must not exceed the {n_steps} steps of the run")
    starts = {"start": warmup, "mid": max(warmup, n_steps // 2 - steps // 2), "end": n_steps - steps}
    marks = {}                                         # step index -> event recorded before that step

    def mark(j):
        if j not in marks:
            marks[j] = torch.cuda.Event(enable_timing=True)
            marks[j].record()

    wanted = {warmup, n_steps}
    for st in starts.values():
        wanted |= {st, st + steps}
    launches = 0
    for j in range(n_steps + 1):
        if j in wanted:
            torch.cuda.synchronize()                   # a window starts and ends with an idle device
            mark(j)
        if j == starts["mid"]:
            K.LAUNCHES[0] = 0
        if j == starts["mid"] + steps:
            launches = K.LAUNCHES[0]
        if j < n_steps:
            tok = argmax(runner.step(entries, device_tokens=tok))     # the sampled tokens never leave the device
    torch.cuda.synchronize()
    out = {name: (marks[st].elapsed_time(marks[st + steps]) / steps, prompt_len + st + steps // 2)
           for name, st in starts.items()}
    out["mean"] = (marks[warmup].elapsed_time(marks[n_steps]) / (n_steps - warmup), (prompt_len + warmup + context) // 2)
    assert runner.length(ids[0]) == context
    for rid in ids:
        runner.end(rid)
    return out, launches


def run_prefill(runner, T, warmup, rng):
    """One prompt of T tokens in one step.  Returns (device ms, submit-to-logits ms), each the median of five:
    the first is the time of the step's kernels alone (tables already on the device); the second runs from
    before the step's tables are built on the host, through their copy to the device, to the logits."""
    import statistics
    import torch
    from kappai_b200 import StepEntry

    V = runner.vocab_size
    dev_ms, all_ms = [], []
    for i in range(warmup + 5):
        toks = rng.integers(0, V, T).tolist()
        ctx, after = runner.prepare([StepEntry("p", toks, [T - 1])])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.run(ctx)
        e1.record()
        torch.cuda.synchronize()
        runner.end("p")
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        runner.step([StepEntry("p", toks, [T - 1])])
        f1.record()
        torch.cuda.synchronize()
        runner.end("p")
        if i >= warmup:
            dev_ms.append(e0.elapsed_time(e1))
            all_ms.append(f0.elapsed_time(f1))
    return statistics.median(dev_ms), statistics.median(all_ms)


def run_e2e(model_dir, batch, prompt_len, steps, warmup, rng, n_layers_note):
    """Decode through Engine.step, the loop a user of the Python entry point runs: every step copies its
    tables (positions, slots, block tables) from pinned host memory and brings the sampled tokens back to the
    host, where the scheduler records them.  (The engine launches the next decode step before it waits for the
    last one's tokens; the token ids themselves go from the sampler to the next step on the device.)"""
    import torch
    from kappai_b200 import Engine, EngineArgs, SamplingParams

    eng = Engine(EngineArgs(model=model_dir, dtype="bfloat16", ctx_size=CONTEXT, max_batch=max(batch, 1),
                            max_step_tokens=PROMPT_LEN, page_size=64, kv_tokens=batch * CONTEXT))
    V = eng.vocab_size
    # room beyond the timed steps: the requests whose prompts ran first decode while the others' prompts run,
    # and nobody may finish (and change the batch) inside the timed region
    sp = SamplingParams(temperature=0.0, n_predict=warmup + steps + 2 * batch + 64)
    for _ in range(batch):
        eng.add_request(rng.integers(0, V, prompt_len).tolist(), sp)
    while any(len(r.output) == 0 for r in eng.requests.values()):
        eng.step()                                     # prefill (untimed)
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n = 0
    for _ in range(steps):
        n += len(eng.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = eng.runner.last_h2d_bytes               # the step's table buffer; greedy sampling copies nothing more
    d2h = batch * 4 + 4                           # the sampled tokens and the step's status word
    eng.shutdown()
    return n / dt, h2d, d2h


def run_workload(name: str, rng_seed: int, time_kernels: bool = False) -> dict:
    """Whole generations through ``Engine`` (scheduler, chunked prefill beside decoding, sampling), timed by
    the wall clock around ``generate``-like stepping, as the reference times its runs (src/context.c:1507-1512,
    1607-1620; src/test/test_bench.c:432-464)."""
    import numpy as np
    import torch
    from kappai_b200 import Engine, EngineArgs, SamplingParams

    if name == "long":
        cfg, seed, n_req, ctx, max_batch = LFM2_2P6B, 3, 16, 32768, 16
        lens = np.random.default_rng(rng_seed).integers(1000, 30001, n_req).tolist()
        n_out, sp_of = 128, lambda i: SamplingParams(temperature=0.0, n_predict=128)
        label = "LFM2-2.6B shape, 16 requests, prompts U[1000,30000], portions of 2048, context 32768, 128 greedy tokens each"
    else:
        cfg, seed, n_req, ctx, max_batch = LFM2_350M, 4, 256, 1024, 256
        lens = np.random.default_rng(rng_seed).integers(16, 513, n_req).tolist()
        n_out, sp_of = 128, lambda i: SamplingParams(temperature=0.8, top_k=40, top_p=0.9, min_p=0.1, seed=4 + i, n_predict=128)
        label = "LFM2-350M shape, 256 requests at once, prompts U[16,512], 128 tokens each at temperature 0.8 (seed 4)"
    model_dir, c = model_folder(cfg, seed, cfg["num_hidden_layers"])
    eng = Engine(EngineArgs(model=model_dir, dtype="bfloat16", ctx_size=ctx, max_batch=max_batch, max_step_tokens=2048,
                            page_size=64, kv_tokens=0, time_kernels=time_kernels))
    rng = np.random.default_rng(rng_seed + 1)
    V = eng.vocab_size
    prompts = [rng.integers(0, V, n).tolist() for n in lens]
    # warm-up: one short generation builds what is built at first use
    eng.generate([prompts[0][:64]], SamplingParams(temperature=0.0, n_predict=4))
    eng.stats = type(eng.stats)()
    torch.cuda.synchronize()
    clocks = ClockSampler()
    clocks.start()
    t0 = time.perf_counter()
    ids = [eng.add_request(p, sp_of(i)) for i, p in enumerate(prompts)]
    first = {}
    n_steps = 0
    while eng.has_work():
        for r in eng.step():
            first.setdefault(r.id, time.perf_counter() - t0)
        n_steps += 1
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    clk = clocks.stop()
    outs = [eng.requests[i].output for i in ids]
    reasons = sorted({eng.finish_reason(i) for i in ids})
    n_prompt, n_new = sum(lens), sum(len(o) for o in outs)
    st = eng.stats
    rec = {"workload": name, "what": label, "impl": "ours", "dtype": "bf16", "seconds": round(dt, 3),
           "prompt_tokens": n_prompt, "new_tokens": n_new, "tokens_per_s": round((n_prompt + n_new) / dt, 1),
           "new_tokens_per_s": round(n_new / dt, 1), "steps": n_steps, "mean_step_ms": round(dt * 1e3 / n_steps, 3),
           "preemptions": eng.scheduler.n_preemptions, "finish_reasons": reasons,
           "mean_ttft_s": round(sum(first.values()) / len(first), 3), "kv_tokens": eng.runner.cache_plan.tokens,
           "graph_captures": eng.runner.graphs.n_captures if eng.runner.graphs else 0,
           "pp_tokens_per_s": round(st.prompt_tokens / st.prompt_seconds, 1) if st.prompt_seconds else None,
           "tg_tokens_per_s": round(st.decode_tokens / st.decode_seconds, 1) if st.decode_seconds else None,
           "clocks": clk}
    if time_kernels:
        # (timed runs launch every kernel on its own, between two events: their throughput is not the engine's)
        print(eng.timer.format(f"workload {name}, every step launched kernel by kernel"), file=sys.stderr)
        rec["timed_kernel_by_kernel"] = True
    eng.shutdown()
    return rec


def run_probe(model_dir, a, rng) -> int:
    """A few eager steps for a profiler: every kernel is a launch of its own (no graph), sizes as in the bench."""
    import torch
    from kappai_b200 import ModelRunner, StepEntry
    from kappai_b200.sampling.sampler import argmax

    B, T = a.batch, a.prompt_len
    runner = ModelRunner(model_dir, dtype="bfloat16", max_tokens=B * CONTEXT, max_requests=B, page_size=64,
                         max_model_len=CONTEXT, cuda_graphs=False)
    V = runner.vocab_size
    if a.probe == "prefill":
        for i in range(a.steps):
            runner.step([StepEntry("p", rng.integers(0, V, T).tolist(), [T - 1])])
            runner.end("p")
    else:
        for i in range(B):
            runner.step([StepEntry(i, rng.integers(0, V, T).tolist(), [])])
        entries = [StepEntry(i, [1], [0]) for i in range(B)]
        for _ in range(a.steps):
            argmax(runner.step(entries))
    torch.cuda.synchronize()
    print(f"probe {a.probe} ok: batch {B}, prompt {T}, {a.steps} steps, {runner.config.num_hidden_layers} layers")
    return 0


def run_timeline(model_dir, a, rng) -> int:
    """The kernels of one captured decode step on the device's own clock: when each one's wait on the kernel
    before it was over, how long until the next one's was, and how early it had become resident (see
    kappai_b200/ops/timeline.py).  Under the trace marks a step runs 10 to 15 % slower."""
    from kappai_b200.ops import timeline
    timeline.enable()
    import torch
    from kappai_b200 import ModelRunner, StepEntry
    from kappai_b200.ops import kernels as K
    from kappai_b200.sampling.sampler import argmax

    B, T = a.batch, a.prompt_len
    runner = ModelRunner(model_dir, dtype="bfloat16", max_tokens=B * CONTEXT, max_requests=B, page_size=64,
                         max_model_len=CONTEXT)
    V = runner.vocab_size
    tok = None
    for i in range(B):
        t = argmax(runner.step([StepEntry(i, rng.integers(0, V, T).tolist(), [T - 1])]))
        tok = t if tok is None else torch.cat([tok, t])
    entries = [StepEntry(i, [0], [0]) for i in range(B)]
    names = None
    for _ in range(6):                                    # the step that is captured logs the names of its launches
        K.LAUNCH_LOG[0] = []
        before = len(runner.graphs.graphs)
        logits = runner.step(entries, device_tokens=tok)
        if len(runner.graphs.graphs) > before:
            names = list(K.LAUNCH_LOG[0])
        K.LAUNCH_LOG[0] = None
        tok = argmax(logits)
    K.LAUNCH_LOG[0] = None
    torch.cuda.synchronize()
    timeline.records()                                    # (clears)
    for _ in range(3):
        tok = argmax(runner.step(entries, device_tokens=tok))
    torch.cuda.synchronize()
    ks = timeline.kernels(timeline.records())
    # the middle one of the three steps: from its first kernel (the embedding) to the next step's
    per_step = len(ks) // 3
    step = ks[per_step:2 * per_step + 1]
    # the names of the captured step's launches, then the sampler's; only if they account for every launch seen
    n_sampling = sum(1 for k in step[:-1] if k["lib"] == "sampling")
    in_graph = per_step - n_sampling - 1                  # (one launch before the graph brings the step's tables)
    print(f"launches: {len(ks)} in three steps, {n_sampling} of the sampler a step, {len(names or [])} names logged",
          file=sys.stderr)
    if names is not None and in_graph > 0 and len(names) >= in_graph:
        # (the capturing call runs the step more than once: the last run)
        names = ["step_tables"] + names[-in_graph:] + ["argmax"] * n_sampling
    else:
        names = None
    span = step[-1]["waited_first"] - step[0]["waited_first"]     # from this step's first kernel to the next step's
    print(f"decode step, batch {B}, context {T + 7}, traced build: {span:.1f} us a step, {per_step} launches")
    print(timeline.table(step, names))
    by = {}
    for i, k in enumerate(step[:-1]):
        w, nxt = k["waited_first"], step[i + 1]["waited_first"]
        if w is None or nxt is None:
            continue
        name = (names[i] if names and i < len(names) else k["lib"])
        got = by.setdefault(name, [0, 0.0])
        got[0] += 1
        got[1] += nxt - w
    total = sum(v[1] for v in by.values())
    print(f"\nby kernel (time on the step's critical path; {total:.1f} us in all):")
    for name, (n, us) in sorted(by.items(), key=lambda kv: -kv[1][1]):
        print(f"  {name:44s} {n:4d} x {us / n:7.2f} us = {us:8.1f} us  {100 * us / total:5.1f} %")
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (0 = all)")
    ap.add_argument("--probe", choices=["decode", "prefill", "timeline"], default=None,
                    help="run a few eager steps (no CUDA graph) of one kind and exit: the small case that a "
                         "profiler is pointed at")
    ap.add_argument("--workload", choices=["long", "many"], default=None,
                    help="run a whole scheduling workload through Engine instead of the default line: 'long' "
                         "(2.6B shape, 16 prompts of 1k to 30k tokens, context 32768) or 'many' (350M shape, 256 requests)")
    ap.add_argument("--time", action="store_true",
                    help="with --workload: launch every kernel on its own between CUDA events and print the device "
                         "time by kernel class (the run's throughput is then not the engine's)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="prompt length of --probe")
    a = ap.parse_args()

    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "System64fumo/kappai is a C program with CPU, Vulkan and OpenGL backends and no Python "
                          "package; it does not install with pip, its build needs json-c which is absent here, and "
                          "it has no CUDA path"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    warmup = max(a.warmup, 3)
    if a.workload:
        print(json.dumps(run_workload(a.workload, 40, a.time)))
        return 0

    import numpy as np
    import torch
    from kappai_b200 import ModelRunner

    pk = peaks()
    n_layers = a.layers or LFM2_1P2B["num_hidden_layers"]
    model_dir, cfg = model_folder(LFM2_1P2B, SEED, n_layers)
    rng = np.random.default_rng(SEED)
    if a.probe == "timeline":
        return run_timeline(model_dir, a, rng)
    if a.probe:
        return run_probe(model_dir, a, rng)
    runner = ModelRunner(model_dir, dtype="bfloat16", max_tokens=64 * CONTEXT, max_requests=64, page_size=64,
                         max_model_len=CONTEXT)
    wbytes = weight_bytes(runner)
    runner_ff = runner.config.intermediate_size

    def window(batch, ms, context):
        by = wbytes + cache_bytes_per_step(runner, batch, context)
        gbs = by / (ms * 1e-3) / 1e9
        return {"tok_s": round(batch * 1e3 / ms, 1), "ms": round(ms, 4), "context": int(context),
                "gb": round(by / 1e9, 3), "frac": round(gbs / pk["hbm_gbs"], 4)}

    clocks = ClockSampler()
    clocks.start()
    win, launches = run_decode(runner, a.batch, PROMPT_LEN, CONTEXT, a.steps, warmup, rng)
    clk = clocks.stop()
    ms, context = win["mid"]
    value = a.batch * 1e3 / ms
    head = window(a.batch, ms, context)

    points = {}
    for b in sorted({1, 8, 64, a.batch}):
        w = win if b == a.batch else run_decode(runner, b, PROMPT_LEN, CONTEXT, a.steps, warmup, rng)[0]
        points[f"decode_b{b}"] = round(b * 1e3 / w["mid"][0], 1)
        for name in ("start", "end", "mean"):
            for k, v in window(b, *w[name]).items():
                points[f"b{b}_{name}_{k}"] = v
        points[f"b{b}_mid_frac"] = window(b, *w["mid"])["frac"]

    pf_ms, pf_all_ms = run_prefill(runner, PROMPT_LEN, warmup, rng)
    flops = 2 * PROMPT_LEN * matrix_params_per_token(runner) + attention_flops(runner, PROMPT_LEN) \
        + 2 * runner.vocab_size * cfg["hidden_size"]
    pf_frac = flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)
    del runner
    torch.cuda.empty_cache()

    e2e, h2d, d2h = run_e2e(model_dir, a.batch, PROMPT_LEN, a.steps, warmup, rng, n_layers)

    rec = {
        "metric": f"decode tok/s at batch {a.batch} (LFM2-1.2B, 2048-token prompts decoding to 4096; the K steps at "
                  "the middle of the run; both ends and the mean in points)",
        "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights (seed 2), uniform random token ids",
        "config": {"model": "LFM2-1.2B shape", "layers": n_layers, "layers_in_config": LFM2_1P2B["num_hidden_layers"],
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"],
                   "ff": runner_ff, "vocab": cfg["vocab_size"], "conv_L_cache": cfg["conv_L_cache"],
                   "global_batch": a.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
                   "context_at_timing": context, "page_size": 64, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights 1.8 GB per step)", "peaks": pk["source"]},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "context": "the first K steps after the prompts (about 2100)"},
        "gpu_launches": int(launches),
        "prefill": {"value": round(PROMPT_LEN * 1e3 / pf_ms, 1), "tokens": PROMPT_LEN, "ms": round(pf_ms, 3),
                    "frac": round(pf_frac, 4), "ms_from_tables_to_logits": round(pf_all_ms, 3),
                    "value_from_tables_to_logits": round(PROMPT_LEN * 1e3 / pf_all_ms, 1), "of": "median of 5"},
        "roofline": {"bound": "hbm", "achieved": round(head["gb"] / (ms * 1e-3), 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": head["frac"], "gb_per_step": head["gb"],
                     "kernel_class_shares": "profiles/decode_step_b8_launches.txt (ncu launch list of one step)"},
        "points": points,
        "clocks": clk,
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
