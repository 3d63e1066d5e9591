"""Whole models at sizes that the tiny configurations do not reach, so that the kernels chosen for real
widths run inside the model and are checked against the plain implementation: head size 64 with a few
thousand tokens (tcgen05 attention for prompt portions, the TMA-fed split kernel for decoded tokens), and
width 512 with decode batches of up to 64 requests (the weight-streaming products in all their forms)."""
import numpy as np
import pytest

from tolerances import tol_for

pytestmark = pytest.mark.gpu

CONFIG = {'architectures': ['Lfm2ForCausalLM'], 'vocab_size': 384, 'hidden_size': 256, 'num_hidden_layers': 3,
          'num_attention_heads': 4, 'num_key_value_heads': 2, 'layer_types': ['conv', 'full_attention', 'full_attention'],
          'max_position_embeddings': 8192, 'norm_eps': 1e-05, 'conv_L_cache': 3, 'conv_bias': False,
          'block_ff_dim': 320, 'block_auto_adjust_ff_dim': False, 'rope_theta': 1000000.0, 'tie_embedding': True}


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    from kappai_b200 import write_random_model
    from plain_lfm2 import PlainLfm2
    d = str(tmp_path_factory.mktemp("long") / "m")
    write_random_model(CONFIG, d, 11)
    return d, PlainLfm2(d)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_in_odd_portions_then_decoding(dtype, model):
    from kappai_b200 import ModelRunner, StepEntry
    from kappai_b200.ops import kernels as K
    d, plain = model
    rng = np.random.default_rng(3)
    T, n_dec = 3000, 6
    toks = rng.integers(0, CONFIG["vocab_size"], T + n_dec).tolist()
    ref = plain.logits(toks)
    r = ModelRunner(d, dtype=dtype, max_tokens=4096, max_requests=2, page_size=64, max_model_len=4096)
    cuts = [0, 129, 700, 701, 1500, 2047, 2048, 2900, T]                 # portions of 129, 571, 1, 799, ... tokens
    tol = tol_for(dtype, ref)
    for a, b in zip(cuts[:-1], cuts[1:]):
        want = sorted({0, (b - a) // 2, b - a - 1})
        lg = r.step([StepEntry("a", toks[a:b], want)]).float().cpu().numpy()
        for j, w in enumerate(want):
            assert np.abs(lg[j] - ref[a + w]).max() <= tol, (dtype, a, b, w)
    for i in range(n_dec):
        lg = r.step([StepEntry("a", [toks[T + i]], [0])]).float().cpu().numpy()
        assert np.abs(lg[0] - ref[T + i]).max() <= tol, (dtype, "decode", i)
    assert K.tc_status() == 0 and K.stream_status() == 0 and K.attention_tc_status() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoded_tokens_beside_prompt_portions(dtype, model):
    """Three requests with caches of different lengths each bring one decoded token while a fourth brings
    portions of its prompt: the decoded rows lead the step (split-key kernel) and the portion follows (tiled
    kernel); then the same with the portion first, where one kernel takes all.  Every row against the plain model."""
    from kappai_b200 import ModelRunner, StepEntry
    from kappai_b200.ops import kernels as K
    d, plain = model
    rng = np.random.default_rng(5)
    V = CONFIG["vocab_size"]
    lens = [1500, 70, 640]
    seqs = [rng.integers(0, V, L + 4).tolist() for L in lens]
    long = rng.integers(0, V, 900).tolist()
    refs = [plain.logits(s) for s in seqs]
    ref_long = plain.logits(long)
    r = ModelRunner(d, dtype=dtype, max_tokens=4096, max_requests=4, page_size=64, max_model_len=4096)
    for i, (s, L) in enumerate(zip(seqs, lens)):
        r.step([StepEntry(i, s[:L], [])])
    cuts = [0, 300, 301, 640, 900]
    for k, (a, b) in enumerate(zip(cuts[:-1], cuts[1:])):
        dec = [StepEntry(i, [s[L + k]], [0]) for i, (s, L) in enumerate(zip(seqs, lens))]
        want = sorted({0, b - a - 1})
        portion = StepEntry("p", long[a:b], want)
        entries = dec + [portion] if k != 2 else [portion] + dec
        lg = r.step(entries).float().cpu().numpy()
        rows = [(refs[i][L + k], (i, k)) for i, L in enumerate(lens)]
        prows = [(ref_long[a + w], ("p", a, w)) for w in want]
        for j, (want_row, what) in enumerate(rows + prows if k != 2 else prows + rows):
            assert np.abs(lg[j] - want_row).max() <= tol_for(dtype, want_row), (dtype, what)
    assert K.tc_status() == 0 and K.stream_status() == 0 and K.attention_tc_status() == 0


WIDE_CONFIG = {'architectures': ['Lfm2ForCausalLM'], 'vocab_size': 640, 'hidden_size': 512, 'num_hidden_layers': 2,
               'num_attention_heads': 8, 'num_key_value_heads': 2, 'layer_types': ['conv', 'full_attention'],
               'max_position_embeddings': 1024, 'norm_eps': 1e-06, 'conv_L_cache': 3, 'conv_bias': False,
               'block_ff_dim': 1024, 'block_auto_adjust_ff_dim': False, 'rope_theta': 10000.0, 'tie_embedding': False}


@pytest.fixture(scope="module")
def wide_model(tmp_path_factory):
    from kappai_b200 import write_random_model
    from plain_lfm2 import PlainLfm2
    d = str(tmp_path_factory.mktemp("wide") / "m")
    write_random_model(WIDE_CONFIG, d, 12)
    return d, PlainLfm2(d)


@pytest.fixture(scope="module")
def wide_bf16_bound(wide_model):
    """The bfloat16 bound at this width, measured as at the LFM2-1.2B shape (tolerances.bf16_bounds_from_ideal): the
    largest error of a row that an ideal implementation with the engine's 16-bit storage points makes, as a fraction
    of the row's standard deviation, times BF16_IDEAL_FACTOR.  (At width 512 the ideal error alone is 4.4 to 4.8 %:
    the 5 % of the tiny models' bound leaves no room for another order of summation.)"""
    from plain_lfm2 import PlainLfm2
    from tolerances import bf16_bounds_from_ideal
    d, plain = wide_model
    emulated = PlainLfm2(d, storage="bfloat16")
    rng = np.random.default_rng(356)
    big = 0.0
    for _ in range(6):
        s = rng.integers(0, WIDE_CONFIG["vocab_size"], 40).tolist()
        big = max(big, bf16_bounds_from_ideal(plain.logits(s), emulated.logits(s))[0])
    return big


@pytest.mark.parametrize("n_req", [3, 20, 40, 64, 100, 256])
def test_decode_batches_at_a_width_the_streaming_kernels_take(n_req, wide_model, wide_bf16_bound):
    """Width 512 (a multiple of the bulk-copy kernel's 512-column chunks): decode steps of 3, 20, 40 and 64
    requests run the weight-streaming products in all their forms (half tile, two, three and four m-tiles,
    16-row weight tiles) inside the model, from captured graphs; steps of 100 and 256 requests run every product
    on the tcgen05 kernel with a short box of rows; every request's logits against the plain model."""
    from kappai_b200 import ModelRunner, StepEntry
    from kappai_b200.ops import kernels as K
    d, plain = wide_model
    rng = np.random.default_rng(100 + n_req)
    V = WIDE_CONFIG["vocab_size"]
    lens = rng.integers(3, 70, n_req).tolist()
    seqs = [rng.integers(0, V, L + 3).tolist() for L in lens]
    refs = [plain.logits(s) for s in seqs]
    r = ModelRunner(d, dtype="bfloat16", max_tokens=n_req * 128, max_requests=n_req, page_size=64, max_model_len=1024)
    for i, (s, L) in enumerate(zip(seqs, lens)):
        r.step([StepEntry(i, s[:L], [])])
    for step in range(3):
        entries = [StepEntry(i, [s[L + step]], [0]) for i, (s, L) in enumerate(zip(seqs, lens))]
        lg = r.step(entries).float().cpu().numpy()
        for i, L in enumerate(lens):
            ref = refs[i][L + step]
            assert np.abs(lg[i] - ref).max() <= wide_bf16_bound * float(ref.std()), (n_req, step, i)
    assert r.graphs.n_replays >= 2
    assert K.tc_status() == 0 and K.stream_status() == 0


def test_a_captured_step_survives_the_growth_of_the_attention_scratch(wide_model):
    """A decode graph keeps the address of the split-key scratch it was captured with.  Capture a graph while
    the scratch is small, make a longer request outgrow it, fill the memory that a freed buffer would have
    returned to with sentinels, then replay the first graph: the sentinels are untouched and the logits right."""
    import torch
    from kappai_b200 import ModelRunner, StepEntry
    d, plain = wide_model
    rng = np.random.default_rng(7)
    V = WIDE_CONFIG["vocab_size"]
    n = 64
    r = ModelRunner(d, dtype="bfloat16", max_tokens=n * 128 + 1024, max_requests=n, page_size=64, max_model_len=1024)
    env = r.model.env

    def batch(lens, tag):
        seqs = [rng.integers(0, V, L + 3).tolist() for L in lens]
        for i, (s, L) in enumerate(zip(seqs, lens)):
            r.step([StepEntry((tag, i), s[:L], [])])
        return seqs

    def decode_and_check(seqs, lens, tag, step):
        lg = r.step([StepEntry((tag, i), [s[L + step]], [0]) for i, (s, L) in enumerate(zip(seqs, lens))])
        lg = lg.float().cpu().numpy()
        for i in (0, 1, n // 2, n - 1):
            ref = plain.logits(seqs[i][:lens[i] + step + 1])[-1]
            assert np.abs(lg[i] - ref).max() <= tol_for("bfloat16", ref), (tag, step, i)

    short = rng.integers(3, 60, n).tolist()
    seqs_a = batch(short, "a")
    decode_and_check(seqs_a, short, "a", 0)                    # (a shape is captured when it comes the second time)
    decode_and_check(seqs_a, short, "a", 1)                    # captures the graph of (64 requests, 8 blocks)
    assert r.graphs.n_captures == 1
    first = env.shared["attn_scratch"]
    for i in range(n):
        r.end(("a", i))
    long = list(short)
    long[0] = 600                                              # one request of 10 blocks: the graph of 16 blocks
    seqs_b = batch(long, "b")
    decode_and_check(seqs_b, long, "b", 0)
    decode_and_check(seqs_b, long, "b", 1)
    assert env.shared["attn_scratch"] is not first and env.shared["attn_scratch"].numel() > first.numel()
    assert any(t is first for t in env.shared["attn_scratch_retired"])
    for i in range(n):
        r.end(("b", i))
    del first
    sentinels = [torch.full((68096,), 7.0, device="cuda") for _ in range(64)]      # what a freed scratch would become
    seqs_c = batch(short, "c")
    decode_and_check(seqs_c, short, "c", 0)                    # replays the first graph
    decode_and_check(seqs_c, short, "c", 1)
    assert r.graphs.n_captures == 2
    torch.cuda.synchronize()
    assert all(bool((t == 7.0).all()) for t in sentinels)


def test_captured_graphs_share_a_pool_and_the_oldest_goes(wide_model):
    """With room for two graphs only, a third shape evicts the one that ran longest ago; a shape that comes back
    is captured again and still right."""
    from kappai_b200 import ModelRunner, StepEntry
    d, plain = wide_model
    rng = np.random.default_rng(9)
    V = WIDE_CONFIG["vocab_size"]
    r = ModelRunner(d, dtype="bfloat16", max_tokens=8 * 128, max_requests=8, page_size=64, max_model_len=128)
    r.graphs.MAX_GRAPHS = 2
    seqs = [rng.integers(0, V, 40).tolist() for _ in range(4)]
    refs = [plain.logits(s) for s in seqs]
    for i, s in enumerate(seqs):
        r.step([StepEntry(i, s[:5 + i], [])])        # (prompts of different lengths: no shape comes thrice in a row)
    fed = [5 + i for i in range(4)]

    def decode(which, steps):
        for _ in range(steps):
            lg = r.step([StepEntry(i, [seqs[i][fed[i]]], [0]) for i in which]).float().cpu().numpy()
            for j, i in enumerate(which):
                assert np.abs(lg[j] - refs[i][fed[i]]).max() <= tol_for("bfloat16", refs[i]), (which, i, fed[i])
                fed[i] += 1

    decode([0, 1, 2, 3], 3)          # shape of 4 requests: captured at its second step
    decode([0, 1, 2], 3)             # 3 requests
    assert r.graphs.n_captures == 2 and r.graphs.n_evicted == 0
    decode([0, 1], 3)                # 2 requests: a third graph, the one of 4 requests goes
    assert r.graphs.n_captures == 3 and r.graphs.n_evicted == 1 and (4, 8) not in r.graphs.graphs
    decode([0, 1, 2, 3], 3)          # and is captured again when it comes back
    assert r.graphs.n_captures == 4 and r.graphs.n_evicted == 2


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_a_prompt_fed_in_equal_portions_beside_decoding_requests_runs_from_a_captured_step(wide_model, dtype):
    """Steps that are not pure decode are captured too where the same shape comes again: two requests decode while
    a third's prompt is fed 16 tokens a step.  The captured steps must give the bits of the steps launched kernel
    by kernel (a second runner without graphs), replays must have happened, and the logits agree with the plain
    model; the portions cross pages and the block table's width grows under way."""
    from kappai_b200 import ModelRunner, StepEntry
    d, plain = wide_model
    rng = np.random.default_rng(12)
    V = WIDE_CONFIG["vocab_size"]
    seqs = [rng.integers(0, V, 60).tolist() for _ in range(2)] + [rng.integers(0, V, 16 * 14).tolist()]
    refs = [plain.logits(s) for s in seqs]

    def run(graphs):
        r = ModelRunner(d, dtype=dtype, max_tokens=1024, max_requests=4, page_size=16, max_model_len=512, cuda_graphs=graphs)
        for i in (0, 1):
            r.step([StepEntry(i, seqs[i][:20], [])])
        out = []
        for t in range(14):
            ent = [StepEntry(i, [seqs[i][20 + t]], [0]) for i in (0, 1)]
            ent.append(StepEntry(2, seqs[2][16 * t:16 * t + 16], [3, 15]))
            out.append(r.step(ent).float().cpu().numpy().copy())
        return out, r

    eager, _ = run(False)
    captured, r = run(True)
    assert r.graphs.n_replays >= 6 and r.graphs.n_step_captures >= 1, (r.graphs.n_replays, r.graphs.n_step_captures)
    for t, (a, b) in enumerate(zip(eager, captured)):
        assert np.array_equal(a, b), f"step {t}: the captured step and the eager step differ"
        for j, (i, pos) in enumerate(((0, 20 + t), (1, 20 + t), (2, 16 * t + 3), (2, 16 * t + 15))):
            assert np.abs(a[j] - refs[i][pos]).max() <= tol_for(dtype, refs[i]), (t, i, pos)
