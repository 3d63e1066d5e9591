#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at the LFM2-1.2B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode step of the whole batch.  The default run has the
layer sizes of the LFM2-1.2B configuration with random weights (seed 2), a
batch of 8 requests, prompts of 2,048 tokens and a context limit of 4,096.
It prints one JSON line:

* ``value``: decoded tokens a second, timed on the device with CUDA events
  around exactly K steps (sampled tokens stay on the device between steps);
* ``e2e``: the same through the Python entry point (``Engine.step``): host
  token ids in, host token ids out, every step;
* ``prefill``: one 2,048-token prompt in one step, with the fraction of the
  bf16 matrix peak;
* ``roofline``: bytes a decode step has to read (every weight once, the cache
  of the live requests) over its time, against the measured copy bandwidth;
* ``points``: decode tokens a second at batch 1 and 64.

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


def run_decode(runner, batch, prompt_len, steps, warmup, rng):
    """Prefill ``batch`` requests, then time ``steps`` decode steps on the device."""
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

    def one_step(tok):
        return argmax(runner.step(entries, device_tokens=tok))     # the sampled tokens never leave the device

    for _ in range(warmup):
        tok = one_step(tok)
    torch.cuda.synchronize()
    K.LAUNCHES[0] = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        tok = one_step(tok)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    launches = K.LAUNCHES[0]
    context = runner.length(ids[0])
    for rid in ids:
        runner.end(rid)
    return ms, launches, context


def run_prefill(runner, T, warmup, rng):
    import torch
    from kappai_b200 import StepEntry

    V = runner.vocab_size
    times = []
    for i in range(warmup + 3):
        toks = rng.integers(0, V, T).tolist()
        ctx, after = runner.prepare([StepEntry("p", toks, [T - 1])])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.run(ctx)
        e1.record()
        torch.cuda.synchronize()
        runner.end("p")
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    return min(times)


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
    d2h = batch * 4
    eng.shutdown()
    return n / dt, h2d, d2h


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


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (0 = all)")
    ap.add_argument("--probe", choices=["decode", "prefill"], default=None,
                    help="run a few eager steps (no CUDA graph) of one kind and exit: the small case that a "
                         "profiler is pointed at")
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

    import numpy as np
    import torch
    from kappai_b200 import ModelRunner

    pk = peaks()
    n_layers = a.layers or LFM2_1P2B["num_hidden_layers"]
    model_dir, cfg = model_folder(LFM2_1P2B, SEED, n_layers)
    rng = np.random.default_rng(SEED)
    if a.probe:
        return run_probe(model_dir, a, rng)
    runner = ModelRunner(model_dir, dtype="bfloat16", max_tokens=64 * CONTEXT, max_requests=64, page_size=64,
                         max_model_len=CONTEXT)
    wbytes = weight_bytes(runner)
    runner_ff = runner.config.intermediate_size

    clocks = ClockSampler()
    clocks.start()
    ms, launches, context = run_decode(runner, a.batch, PROMPT_LEN, a.steps, warmup, rng)
    clk = clocks.stop()
    value = a.batch * 1e3 / ms
    step_bytes = wbytes + cache_bytes_per_step(runner, a.batch, context - a.steps // 2)
    achieved = step_bytes / (ms * 1e-3) / 1e9

    points = {}
    for b in (1, 64):
        pms, _, _ = run_decode(runner, b, PROMPT_LEN, max(8, a.steps // 2), warmup, rng)
        points[f"decode_b{b}"] = round(b * 1e3 / pms, 1)

    pf_ms = run_prefill(runner, PROMPT_LEN, warmup, rng)
    flops = 2 * PROMPT_LEN * matrix_params_per_token(runner) + attention_flops(runner, PROMPT_LEN) \
        + 2 * runner.vocab_size * cfg["hidden_size"]
    pf_frac = flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)
    del runner
    torch.cuda.empty_cache()

    e2e, h2d, d2h = run_e2e(model_dir, a.batch, PROMPT_LEN, a.steps, warmup, rng, n_layers)

    rec = {
        "metric": "decode tok/s at batch 8 (LFM2-1.2B, context 2048->4096)", "value": round(value, 1),
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
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches),
        "prefill": {"value": round(PROMPT_LEN * 1e3 / pf_ms, 1), "tokens": PROMPT_LEN, "ms": round(pf_ms, 3),
                    "frac": round(pf_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clk,
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
