"""The engine through its entry points: greedy generation against the plain
implementation, long decoding, first tokens, reuse of slots and pages,
preemption by recompute, seeded sampling, the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tolerances import tol_for

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def check_greedy(plain, prompt, out, dtype):
    """Each generated token is the plain argmax, or a near tie of it, given the tokens before it."""
    seq = list(prompt)
    all_logits = plain.logits(seq + list(out))
    for j, t in enumerate(out):
        lg = all_logits[len(prompt) + j - 1]
        best = int(np.argmax(lg))
        if t != best:
            assert lg[best] - lg[t] <= 2 * tol_for(dtype, lg), (j, t, best, lg[best] - lg[t])


def engine(model_dir, dtype="float32", **kw):
    from kappai_b200 import Engine, EngineArgs
    args = dict(model=model_dir, dtype=dtype, max_batch=4, max_step_tokens=32, page_size=16, kv_tokens=2048)
    args.update(kw)
    return Engine(EngineArgs(**args))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_matches_plain(name, dtype, model_dirs, plain_models):
    from kappai_b200 import SamplingParams
    plain = plain_models[name]
    V = plain.cfg["vocab_size"]
    rng = np.random.default_rng(20)
    lens, n_new = ([5, 17, 33], 16) if name == "A" else ([1, 9, 64, 130], 24)      # the workloads of the two configs
    prompts = [rng.integers(0, V, n).tolist() for n in lens]
    eng = engine(model_dirs[name], dtype, max_step_tokens=16)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, n_predict=n_new))
    assert [len(o) for o in outs] == [n_new] * len(prompts)
    for p, o in zip(prompts, outs):
        check_greedy(plain, p, o, dtype)
    assert eng.runner.cache.slots.n_free == 4 and all(p.n_free == p.n_pages for p in eng.runner.cache.pools.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, model_dirs, plain_models):
    """400 tokens decoded one by one after a 3-token prompt; logits at every step against plain."""
    from kappai_b200 import ModelRunner, StepEntry
    plain = plain_models["C"]
    rng = np.random.default_rng(21)
    toks = rng.integers(0, plain.cfg["vocab_size"], 403).tolist()
    ref = plain.logits(toks)
    r = ModelRunner(model_dirs["C"], dtype=dtype, max_tokens=512, page_size=32)
    got = [r.step([StepEntry("a", toks[:3], [0, 1, 2])]).cpu().double().numpy()]
    for t in toks[3:]:
        got.append(r.step([StepEntry("a", [t], [0])]).cpu().double().numpy())
    got = np.concatenate(got)
    err = np.abs(got - ref).max(axis=1)
    tol = tol_for(dtype, ref)
    assert err.max() <= tol, f"first wrong position {int(np.argmax(err > tol))}: {err.max()} > {tol}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens(dtype, model_dirs, plain_models):
    """Positions 0, 1, 2 of a sequence, fed one by one, two at once, and as prompts of length 1, 2, 3."""
    from kappai_b200 import ModelRunner, StepEntry
    for name in ("A", "B"):
        plain = plain_models[name]
        toks = [7, 200, 31]
        ref = plain.logits(toks)
        tol = tol_for(dtype, ref)
        r = ModelRunner(model_dirs[name], dtype=dtype, max_tokens=256, page_size=16)
        for cut in ([1, 1, 1], [2, 1], [1, 2], [3]):
            got, i = [], 0
            for n in cut:
                got.append(r.step([StepEntry("x", toks[i:i + n], list(range(n)))]).cpu().double().numpy())
                i += n
            r.end("x")
            assert np.abs(np.concatenate(got) - ref).max() <= tol, (name, cut)


def test_reused_slot_and_pages_give_the_same_bits(model_dirs):
    """After other requests have used and left the slot and the pages, a request
    replayed gives bit-identical logits (no stale state or keys leak in)."""
    from kappai_b200 import ModelRunner, StepEntry
    rng = np.random.default_rng(22)
    for dtype in ("float32", "bfloat16"):
        r = ModelRunner(model_dirs["B"], dtype=dtype, max_tokens=128, page_size=16, max_requests=2)
        toks = rng.integers(0, 512, 60).tolist()
        run = lambda rid: torch.cat([r.step([StepEntry(rid, toks[:37], list(range(37)))]),
                                     r.step([StepEntry(rid, toks[37:], list(range(23)))])])
        first = run("a")
        r.end("a")
        for k in range(3):                                  # dirty every page and both slots
            other = rng.integers(0, 512, 96).tolist()
            r.step([StepEntry(f"o{k}", other, []), StepEntry(f"p{k}", other[:20], [])])
            r.end(f"o{k}"); r.end(f"p{k}")
        again = run("b")
        assert torch.equal(first, again)


def test_preemption_recomputes_and_gives_the_same_tokens(model_dirs, plain_models):
    from kappai_b200 import SamplingParams
    plain = plain_models["B"]
    rng = np.random.default_rng(23)
    prompts = [rng.integers(0, 512, n).tolist() for n in (40, 33, 50, 21)]
    sp = SamplingParams(temperature=0.0, n_predict=40)
    roomy = engine(model_dirs["B"], "float32", kv_tokens=2048)
    want = roomy.generate(prompts, sp)
    assert roomy.scheduler.n_preemptions == 0
    tight = engine(model_dirs["B"], "float32", kv_tokens=16 * 14)        # 14 pages for four requests of up to 90 tokens
    got = tight.generate(prompts, sp)
    assert tight.scheduler.n_preemptions > 0
    assert [tight.finish_reason(i) for i in range(4)] == ["length"] * 4
    # recomputed in other portions and beside other requests, the 32-bit path gives the same bits, so the same tokens
    assert got == want
    for p, b in zip(prompts, got):
        check_greedy(plain, p, b, "float32")
    tight.runner.cache.check()


def test_request_too_large_for_the_pool_ends_with_out_of_memory(model_dirs):
    from kappai_b200 import SamplingParams
    eng = engine(model_dirs["B"], "float32", kv_tokens=64, max_step_tokens=64)
    a = eng.add_request(list(range(60)), SamplingParams(temperature=0.0, n_predict=30))
    b = eng.add_request(list(range(10)), SamplingParams(temperature=0.0, n_predict=3))
    while eng.has_work():
        eng.step()
    assert eng.finish_reason(a) == "out_of_memory" and len(eng.requests[a].output) == 5      # 64 tokens fit, the 65th does not
    assert eng.finish_reason(b) == "length" and len(eng.requests[b].output) == 3


def test_seeded_sampling_does_not_depend_on_the_batch(model_dirs):
    from kappai_b200 import SamplingParams
    rng = np.random.default_rng(24)
    prompts = [rng.integers(0, 256, n).tolist() for n in (12, 30, 7)]
    sp = lambda seed: SamplingParams(temperature=0.8, top_k=40, top_p=0.9, min_p=0.1, seed=seed, n_predict=12)
    eng = engine(model_dirs["A"], "float32")
    together = eng.generate(prompts, [sp(5), sp(6), sp(7)])
    alone = [engine(model_dirs["A"], "float32").generate([p], sp(5 + i))[0] for i, p in enumerate(prompts)]
    assert together == alone
    assert engine(model_dirs["A"], "float32").generate(prompts[:1], sp(99))[0] != alone[0]
    # sampling with another seed, and greedy decoding, each take another path through the same logits
    greedy = engine(model_dirs["A"], "float32").generate(prompts[:1], SamplingParams(temperature=0.0, n_predict=12))[0]
    assert greedy != alone[0] and greedy != engine(model_dirs["A"], "float32").generate(prompts[:1], sp(99))[0]


def test_sampling_over_a_vocabulary_of_65536_in_the_engine(tmp_path):
    """Temperature sampling inside the engine at the vocabulary of the real models (the sampler's two-stage
    kernels): requests with seeds sampled together give what each gives alone, with and without the filters."""
    from kappai_b200 import SamplingParams, write_random_model
    cfg = dict(architectures=["Lfm2ForCausalLM"], vocab_size=65536, hidden_size=64, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, layer_types=["conv", "full_attention"],
               max_position_embeddings=256, norm_eps=1e-5, conv_L_cache=3, conv_bias=False, block_ff_dim=128,
               block_auto_adjust_ff_dim=False, rope_theta=10000.0, tie_embedding=True)
    d = write_random_model(cfg, str(tmp_path / "v64k"), 8)
    rng = np.random.default_rng(25)
    prompts = [rng.integers(0, 65536, n).tolist() for n in (12, 30, 7)]
    sps = [SamplingParams(temperature=0.8, top_k=40, top_p=0.9, min_p=0.1, seed=5, n_predict=10),
           SamplingParams(temperature=1.3, top_k=0, top_p=1.0, min_p=0.0, seed=6, n_predict=10),      # no filter: the whole vocabulary
           SamplingParams(temperature=0.8, top_k=0, top_p=0.95, min_p=0.0, seed=7, n_predict=10)]
    together = engine(d, "float32").generate(prompts, sps)
    alone = [engine(d, "float32").generate([p], sp)[0] for p, sp in zip(prompts, sps)]
    assert together == alone
    assert all(0 <= t < 65536 for o in together for t in o) and len({t for o in together for t in o}) > 20
    # the unfiltered request samples from a flat distribution: its tokens are not the greedy ones
    greedy = engine(d, "float32").generate(prompts[1:2], SamplingParams(temperature=0.0, n_predict=10))[0]
    assert greedy != together[1]


def test_a_cache_that_cannot_fit_is_refused_with_the_figures(model_dirs):
    """The failsafe of src/context.c:395-429,479-491: refuse before allocating, with a sentence."""
    from kappai_b200.engine.runner import EngineError
    from kappai_b200 import Engine, EngineArgs
    small = lambda: 3 << 20                                                   # pretend 3 MB are free
    with pytest.raises(EngineError, match=r"needs .* MB .* but only .* MB can be used .* refusing to run"):
        Engine(EngineArgs(model=model_dirs["B"], dtype="float32", max_batch=4, kv_tokens=1 << 16), free_memory=small)
    # with the size left open the engine takes what fits: fewer tokens than 4 x 256, at least one request of 256
    eng = Engine(EngineArgs(model=model_dirs["B"], dtype="float32", max_batch=4, page_size=16),
                 free_memory=lambda: 600 << 10)
    tokens = eng.runner.cache_plan.tokens
    assert 256 <= tokens < 4 * 256 and eng.runner.cache_plan.cache_bytes <= (600 << 10)
    with pytest.raises(EngineError, match="not even one request"):
        Engine(EngineArgs(model=model_dirs["B"], dtype="float32", max_batch=4), free_memory=lambda: 1 << 16)
    with pytest.raises(EngineError, match="max_step_tokens"):
        Engine(EngineArgs(model=model_dirs["B"], max_step_tokens=70000))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_launched_ahead_change_nothing(dtype, model_dirs):
    """The engine launches the next decode step before it has read the last one's tokens.  The same workload
    with and without that: requests that end by an end-of-sequence token while a step with them is under way,
    by their length, a request that arrives in the middle, one that is aborted, seeded sampling; the tokens,
    the reasons and the state of the cache at the end are the same."""
    from kappai_b200 import SamplingParams
    rng = np.random.default_rng(31)
    prompts = [rng.integers(0, 512, n).tolist() for n in (9, 40, 3, 25)]
    late = rng.integers(0, 512, 12).tolist()
    sps = [SamplingParams(temperature=0.0, n_predict=30), SamplingParams(temperature=0.0, n_predict=17),
           SamplingParams(temperature=0.9, top_k=50, seed=4, n_predict=26), SamplingParams(temperature=0.0, n_predict=60)]

    def run(look_ahead, eos):
        eng = engine(model_dirs["B"], dtype, look_ahead=look_ahead, max_step_tokens=64)
        eng.scheduler.eos_token_id = eos
        ids = [eng.add_request(p, sp) for p, sp in zip(prompts, sps)]
        n = 0
        while eng.has_work():
            eng.step()
            n += 1
            if n == 8:
                ids.append(eng.add_request(late, SamplingParams(temperature=0.0, n_predict=9)))
            if n == 22:
                eng.abort(ids[3])
        eng.runner.cache.check()
        assert eng.runner.cache.slots.n_free == 4
        outs = [eng.requests[i].output for i in ids]
        return outs, [eng.finish_reason(i) for i in ids], eng.n_launched_ahead

    plain_outs, _, _ = run(False, None)
    eos = plain_outs[0][11]                                  # a token the first request meets on its way
    want = run(False, eos)
    got = run(True, eos)
    assert want[2] == 0 and got[2] > 10
    assert got[:2] == want[:2]
    assert "eos" in want[1] and "length" in want[1] and "aborted" in want[1]


def test_context_full_and_bad_requests(model_dirs):
    from kappai_b200 import SamplingParams
    eng = engine(model_dirs["A"], "float32", ctx_size=40)
    rid = eng.add_request(list(range(30)), SamplingParams(temperature=0.0, n_predict=-1))
    while eng.has_work():
        eng.step()
    assert eng.finish_reason(rid) == "context_full" and len(eng.requests[rid].output) == 10
    with pytest.raises(ValueError, match="vocabulary"):
        eng.add_request([1, 2, 999], None)
    with pytest.raises(ValueError, match="limit"):
        eng.add_request(list(range(40)), None)
    with pytest.raises(ValueError, match="prompt token"):
        eng.add_request([], None)


def test_command_line(model_dirs, tmp_path):
    from kappai_b200 import SamplingParams
    want = engine(model_dirs["A"], "bfloat16", max_batch=64, max_step_tokens=2048, page_size=64, kv_tokens=0) \
        .generate([[5, 17, 3, 200]], SamplingParams(temperature=0.0, n_predict=6))[0]
    cmd = [sys.executable, "-m", "kappai_b200.cli", "-m", model_dirs["A"], "-p", "5,17,3,200", "-n", "6", "-t", "0",
           "--metrics", "pp,tg,ttft"]
    p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(t) for t in p.stdout.split()] == want
    assert "TG:" in p.stderr and "t/s" in p.stderr
    # random-weights mode writes a model folder and runs it; the fp32 flag; exit code 2 when the context fills
    cfgp = tmp_path / "c.json"
    with open(os.path.join(model_dirs["B"], "config.json")) as f:
        cfgp.write_text(f.read())
    out = tmp_path / "rw"
    cmd = [os.path.join(ROOT, "bin", "kappai-cli"), "--random-weights", str(cfgp), "-s", "3", "-m", str(out), "--fp32",
           "-c", "12", "-t", "0", "7 8 9"]
    p = subprocess.run(cmd, cwd=str(tmp_path), capture_output=True, text=True, timeout=300)
    assert p.returncode == 2, p.stderr[-2000:]
    assert len(p.stdout.split()) == 9
    assert os.path.isfile(out / "model.safetensors") and os.path.isfile(out / "config.json")


def test_time_debug_forward_and_debug_flags(model_dirs, plain_models):
    """--time prints device time by kernel class, --debug-forward the statistics of the residual behind every
    layer of the first step (the plain model's, here) and the top logits at every sample, --debug a line a step."""
    import re
    prompt = [5, 17, 3, 200, 9, 41, 7]
    cmd = [sys.executable, "-m", "kappai_b200.cli", "-m", model_dirs["A"], "-p", ",".join(map(str, prompt)), "-n", "4",
           "-t", "0", "--fp32", "--time", "--debug-forward", "--debug"]
    p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    err = p.stderr
    # per-layer statistics against the plain model
    trace = []
    plain_models["A"].hidden(prompt, trace)
    lines = [l for l in err.splitlines() if l.startswith("[debug-forward]") and ("layer" in l or "embedding" in l)]
    assert len(lines) == len(trace) == 5, err[-2000:]
    for line, x in zip(lines, trace):
        got = {k: float(v) for k, v in re.findall(r"(min|max|mean|rms) ([-+0-9.e]+)", line)}
        for k, want in (("min", x.min()), ("max", x.max()), ("mean", x.mean()), ("rms", np.sqrt((x * x).mean()))):
            assert abs(got[k] - want) <= 1e-5 + 1e-4 * abs(want), (line, k, want)
    assert "(shortconv)" in lines[1] and "(attention)" in lines[2]
    tops = [l for l in err.splitlines() if "top logits:" in l]
    assert len(tops) == 4
    first = int(re.search(r"top logits: \[(\d+)\]=", tops[0]).group(1))
    assert first == int(p.stdout.split()[0]) == int(np.argmax(plain_models["A"].logits(prompt)[-1]))
    # the kernel classes with their times
    assert "[profile]" in err and re.search(r"gemm_nt_simt 192x64\s+[0-9.]+\s+\d+", err), err[-3000:]
    assert "rmsnorm_rows" in err and "argmax_rows" in err and "TFLOP/s" in err
    # one line a step
    steps = [l for l in err.splitlines() if l.startswith("[debug] step")]
    assert len(steps) == 4 and "0:0+7" in steps[0] and "finished: length" in steps[-1], steps


def test_no_cuda_device_is_refused(model_dirs):
    from kappai_b200.engine.runner import EngineError, ModelRunner
    with pytest.raises(EngineError, match="CUDA"):
        ModelRunner(model_dirs["A"], device="cpu")
