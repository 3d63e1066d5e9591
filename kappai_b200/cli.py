"""Command line and the Python entry point, in the reference's manner.

The reference's entry point is ``engine_init(ctx, args, argc, argv)`` ->
``engine_run`` -> ``engine_shutdown`` (src/engine.h:12-17, src/cli/main.c:3-17)
with a table-driven flag parser (src/config.c:403-447).  The same three calls
exist here; flags keep the reference's names and meanings where it has them
(-m, -c, -p, -n, -t, -k, -P, -M, --repeat-penalty, --repeat-last-n, -s,
--metrics, --stream, --time, --debug-forward, --debug).  There is no tokenizer in the engine:
a prompt is a list of token ids ("5,17,3" or "5 17 3") and so is the output.

    python -m kappai_b200.cli -m MODEL_DIR -p "5,17,3" -n 16 -t 0
    python -m kappai_b200.cli --random-weights config.json -s 2 -m /tmp/model -p "1 2 3"
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import time
from typing import List, Optional, Sequence, Tuple

from .engine.engine import Engine, EngineArgs
from .sampling.params import SamplingParams

ENGINE_EXIT = 1                    # src/engine.h:7-10
ENGINE_EXIT_CONTEXT_FULL = 2

_TRUE, _FALSE = ("yes", "on", "true", "1"), ("no", "off", "false", "0")     # src/config.c:37-42


def parse_bool(s: str) -> bool:
    v = s.strip().lower()
    if v in _TRUE:
        return True
    if v in _FALSE:
        return False
    raise argparse.ArgumentTypeError(f"expected one of {'/'.join(_TRUE + _FALSE)}, got '{s}'")


def parse_tokens(s: str) -> List[int]:
    parts = [p for p in re.split(r"[,\s]+", s.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise argparse.ArgumentTypeError(f"a prompt is a list of token ids, got '{s}'") from None


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(
        prog="kappai-b200", formatter_class=argparse.RawDescriptionHelpFormatter,
        description="Generate token ids with an LFM2 model on one B200.")
    g = ap.add_argument_group("Engine")
    g.add_argument("-m", "--model", required=True, help="model folder (config.json + model.safetensors)")
    g.add_argument("-c", "--ctx-size", type=int, default=0, help="context size (0 = from model)")
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                   help="bfloat16 (default) or float32: the whole model in true 32-bit")
    g.add_argument("--fp32", action="store_true", help="same as --dtype float32")
    g.add_argument("--max-batch", type=int, default=64, help="requests that run together (default 64)")
    g.add_argument("--max-step-tokens", type=int, default=2048, help="token budget of one step (default 2048)")
    g.add_argument("--page-size", type=int, default=64, help="tokens in a cache page (default 64)")
    g.add_argument("--kv-tokens", type=int, default=0, help="tokens the cache pools hold (0 = max-batch x ctx)")
    g.add_argument("--device", default="cuda:0", help="compute device (default: cuda:0)")
    g.add_argument("--random-weights", metavar="CONFIG", help="write a model folder with random weights from this "
                   "config.json into --model first (seed: -s)")
    g.add_argument("--stream", type=parse_bool, nargs="?", const=True, default=True,
                   help="print tokens as they are generated (default: on)")
    g.add_argument("--metrics", default="pp,tg", help="comma-separated metrics after generation: pp,tg,ttft")
    b = ap.add_argument_group("LLM behavior")
    b.add_argument("-p", "--prompt", action="append", type=parse_tokens, default=None,
                   help="prompt as token ids, e.g. \"5,17,3\" (repeat for several requests)")
    b.add_argument("--tokens-file", help="file with one prompt (token ids) a line")
    b.add_argument("-n", "--n-predict", type=int, default=-1, help="max tokens to generate (-1 = unlimited)")
    b.add_argument("-t", "--temperature", type=float, default=0.80, help="sampling temperature (default 0.80, 0.0 = greedy)")
    b.add_argument("-k", "--top-k", type=int, default=40, help="top-k sampling (default 40, 0 = disabled)")
    b.add_argument("-P", "--top-p", type=float, default=0.90, help="top-p sampling (default 0.90, 1.0 = disabled)")
    b.add_argument("-M", "--min-p", type=float, default=0.10, help="min-p sampling (default 0.10, 0.0 = disabled)")
    b.add_argument("--repeat-penalty", type=float, default=1.0, help="repetition penalty (default 1.0 = disabled)")
    b.add_argument("--repeat-last-n", type=int, default=64, help="last-n tokens considered by repeat penalty (default 64)")
    b.add_argument("-s", "--seed", type=int, default=0, help="RNG seed (0 = random)")
    d = ap.add_argument_group("Tools / debug")
    d.add_argument("--time", action="store_true", help="print device time by kernel class after generation")
    d.add_argument("--debug-forward", action="store_true",
                   help="print per-layer activation stats for the first step and the top logits at every sample")
    d.add_argument("--debug", action="store_true", help="enable debug-level logging (one line a step)")
    ap.add_argument("positional_prompt", nargs="?", type=parse_tokens, help="prompt (token ids) if -p is not given")
    return ap


def engine_init(argv: Optional[Sequence[str]] = None) -> Tuple[Engine, argparse.Namespace]:
    """Parse flags, load the model, make the engine (src/engine.c:410-435)."""
    a = build_parser().parse_args(argv)
    if a.fp32:
        a.dtype = "float32"
    if a.random_weights:
        from .weights.random_init import write_random_model

        with open(a.random_weights, "r", encoding="utf-8") as f:
            write_random_model(json.load(f), a.model, a.seed)
    if a.debug:
        import logging

        logging.basicConfig(stream=sys.stderr, format="[debug] %(message)s")
        logging.getLogger("kappai_b200").setLevel(logging.DEBUG)
    eng = Engine(EngineArgs(model=a.model, dtype=a.dtype, ctx_size=a.ctx_size, max_batch=a.max_batch,
                            max_step_tokens=a.max_step_tokens, page_size=a.page_size, kv_tokens=a.kv_tokens,
                            device=a.device, time_kernels=a.time, debug_forward=a.debug_forward))
    return eng, a


def engine_run(eng: Engine, a: argparse.Namespace) -> int:
    """One-shot generation for the given prompts (src/engine.c:162-196,450-468).
    Returns 0, or ENGINE_EXIT_CONTEXT_FULL if a request ran into the context limit."""
    prompts = list(a.prompt or [])
    if a.tokens_file:
        with open(a.tokens_file, "r", encoding="utf-8") as f:
            prompts += [parse_tokens(line) for line in f if line.strip()]
    if not prompts and a.positional_prompt:
        prompts.append(a.positional_prompt)
    if not prompts:
        print("no prompt given (-p \"5,17,3\")", file=sys.stderr)
        return ENGINE_EXIT
    sp = SamplingParams(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, min_p=a.min_p,
                        repeat_penalty=a.repeat_penalty, repeat_last_n=a.repeat_last_n, seed=a.seed,
                        n_predict=a.n_predict)
    single = len(prompts) == 1
    t0 = time.perf_counter()
    first = [None]

    def on_token(rid, tok):
        if first[0] is None:
            first[0] = time.perf_counter() - t0
        if a.stream and single:
            sys.stdout.write(f"{tok} ")
            sys.stdout.flush()

    outs = eng.generate(prompts, sp, on_token)
    total = time.perf_counter() - t0
    if a.stream and single:
        sys.stdout.write("\n")
    else:
        for o in outs:
            print(" ".join(str(t) for t in o))
    st = eng.stats
    parts = []
    wanted = [m.strip() for m in a.metrics.split(",") if m.strip()]
    if "pp" in wanted and st.prompt_seconds > 0:
        parts.append(f"PP: {st.prompt_tokens / st.prompt_seconds:.2f} t/s")
    if "tg" in wanted and st.decode_seconds > 0:
        parts.append(f"TG: {st.decode_tokens / st.decode_seconds:.2f} t/s")
    if "ttft" in wanted and first[0] is not None:
        parts.append(f"TTFT: {first[0] * 1e3:.1f} ms")
    if parts:
        print("[ " + " | ".join(parts) + " ]", file=sys.stderr)       # src/context.c:1519-1568
    if a.time:
        # device time by kernel class, in the manner of the reference's profile report (src/profile.c:65-110)
        print(eng.timer.format(f"{st.n_steps} steps, wall {total * 1e3:.1f} ms, preemptions "
                               f"{eng.scheduler.n_preemptions}"), file=sys.stderr)
    full = any(eng.finish_reason(i) == "context_full" for i in eng.requests)
    return ENGINE_EXIT_CONTEXT_FULL if full else 0


def engine_shutdown(eng: Engine) -> None:
    eng.shutdown()


def main(argv: Optional[Sequence[str]] = None) -> int:
    eng, a = engine_init(argv)
    try:
        return engine_run(eng, a)
    finally:
        engine_shutdown(eng)


if __name__ == "__main__":
    sys.exit(main())
