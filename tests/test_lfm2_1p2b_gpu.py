"""The LFM2-1.2B shape itself (hidden 2048, feed-forward 5632, vocabulary 65536, 32 query and 8 kv heads of
64, random weights from seed 2): the sizes the benchmark times, checked.

1. The float32 path of the engine at the real layer widths against the plain implementation: four layers
   (conv, conv, attention, conv), so that the float64 plain model stays a matter of seconds.
2. All sixteen layers through ``bin/trace_run`` in the four ways of cutting the work (whole; the last 32 tokens
   one by one; portions of changing size, among them one of two tokens, one of more than 128 and one of more
   than 1024 rows; mixed, up to four requests live, with so few pages that they are used again): bfloat16
   against the engine's own float32 run of the same trace, within the bound stated for sixteen layers, the
   greedy token equal or a near tie by that bound; and float32 equal to itself, bit for bit, across the cuts.
   A kernel whose bounded wait gives up ends ``trace_run`` with an error, so a green run also says that
   every status word stayed zero.

The reference's counterparts are its chunking-equivalence tests on the real layer stack
(src/test/test_hybrid.c:153-387, src/test/test_arch.c:1465-1481)."""
import numpy as np
import pytest

import replay_util as R
from tiny_configs import LFM2_1P2B, LFM2_1P2B_SEED
from tolerances import bf16_bounds_for, fp32_tol_at_width

pytestmark = pytest.mark.gpu


def test_float32_path_at_the_real_widths_against_plain(tmp_path):
    from kappai_b200 import ModelRunner, StepEntry, write_random_model
    from plain_lfm2 import PlainLfm2
    cfg = dict(LFM2_1P2B, num_hidden_layers=4, layer_types=["conv", "conv", "full_attention", "conv"])
    d = str(tmp_path / "m4")
    write_random_model(cfg, d, LFM2_1P2B_SEED)
    rng = np.random.default_rng(41)
    toks = rng.integers(0, cfg["vocab_size"], 96).tolist()
    ref = PlainLfm2(d).logits(toks)
    r = ModelRunner(d, dtype="float32", max_tokens=256, max_requests=2, page_size=64)
    # most of it in one step, two tokens, then the rest one by one
    got = [r.step([StepEntry("a", toks[:81], list(range(81)))]), r.step([StepEntry("a", toks[81:83], [0, 1])])]
    got = [g.double().cpu().numpy() for g in got]
    for t in toks[83:]:
        got.append(r.step([StepEntry("a", [t], [0])]).double().cpu().numpy())
    r.check_status()
    err = np.abs(np.concatenate(got) - ref).max(axis=1)
    tol = fp32_tol_at_width(cfg["hidden_size"])
    print(f"float32, 4 layers at the 1.2B widths: worst |error| {err.max():.3e} (bound {tol:.3e}), "
          f"logits std {ref.std():.3f}")
    assert err.max() <= tol, f"first wrong position {int(np.argmax(err > tol))}: {err.max():.3e} > {tol:.3e}"


LENGTHS = {"r300": 316, "r700": 716, "r1100": 1116, "s90": 106, "s150": 166}     # prompt + 16 decoded tokens
PROMPT = {k: v - 16 for k, v in LENGTHS.items()}


def build_trace(reqs, max_tokens):
    """The four families over the same requests.  Wanted rows are thinned out (a row is 256 KB): every 41st
    position and the last 17 of the whole run, every portion's ends, each token decoded one by one."""
    tr = R.Trace()
    big = {k: reqs[k] for k in ("r300", "r700", "r1100")}
    for rid, toks in big.items():                                   # whole (1116 rows in one step: more than 1024)
        n = len(toks)
        tr.add([(rid, toks, sorted(set(range(0, n, 41)) | set(range(n - 17, n))))], end=[rid])
    R.last_decoded(tr, big, n_last=32)
    sizes = {"r300": [7, 2, 150, 3, 2, 64, 2], "r700": [2, 130, 5, 2, 300, 2, 129, 16], "r1100": [1030, 2, 7, 3, 2, 40]}
    for rid, toks in big.items():                                   # portions of changing size
        i, k = 0, 0
        while i < len(toks):
            n = min(sizes[rid][k % len(sizes[rid])], len(toks) - i)
            if len(toks) - i - n == 1:
                n += 1
            k += 1
            tr.add([(rid, toks[i:i + n], sorted({0, n // 2, n - 1}))], end=[rid] if i + n == len(toks) else [])
            i += n
    b = len(tr.steps)
    order = {k: reqs[k] for k in ("s90", "r300", "s150", "r700", "r1100")}       # who starts when others end
    R.mixed(tr, order, PROMPT, seed=5, max_live=4, page=64, max_tokens=max_tokens)
    assert max(len(s["entries"]) for s in tr.steps[b:]) >= 3
    assert any(len(e["tokens"]) == 1 for s in tr.steps[b:] for e in s["entries"] if len(s["entries"]) > 1)
    return tr


def test_all_sixteen_layers_bfloat16_against_float32_in_every_cut(tmp_path):
    from kappai_b200 import write_random_model
    d = str(tmp_path / "m16")
    write_random_model(LFM2_1P2B, d, LFM2_1P2B_SEED)
    rng = np.random.default_rng(42)
    reqs = {rid: rng.integers(0, LFM2_1P2B["vocab_size"], n).tolist() for rid, n in LENGTHS.items()}
    max_tokens = 1152 + 2 * 64                                      # the longest request and two pages more
    tr = build_trace(reqs, max_tokens)
    out32 = R.run_trace(d, "float32", tr, str(tmp_path / "o32"), max_tokens, timeout=1200)
    out16 = R.run_trace(d, "bfloat16", tr, str(tmp_path / "o16"), max_tokens, timeout=1200)
    for o in ("o32", "o16"):
        stats = R.cache_stats(str(tmp_path / o))
        assert all(g["reused"] > 0 for g in stats.values()), stats

    # float32: the same bits for a (request, position) however the work was cut
    places32 = R.rows_by_place(tr, out32)
    n_multi = 0
    for place, rows in places32.items():
        n_multi += len(rows) > 1
        for r in rows[1:]:
            assert np.array_equal(rows[0], r), f"float32 logits of {place} differ between cuts"
    assert n_multi > 100

    # bfloat16 against float32, row by row, in every family
    rel, rel_rms = bf16_bounds_for(LFM2_1P2B["num_hidden_layers"], LFM2_1P2B["vocab_size"])
    worst, worst_rms, n_rows, flips = 0.0, 0.0, 0, []
    for st, rows in zip(tr.steps, tr.rows):
        for j, place in enumerate(rows):
            a, b = out16[st["step"]][j].astype(np.float64), out32[st["step"]][j].astype(np.float64)
            tol = rel * float(b.std())
            err = float(np.abs(a - b).max())
            rms = float(np.sqrt(np.mean((a - b) ** 2)))
            worst, worst_rms = max(worst, err / float(b.std())), max(worst_rms, rms / float(b.std()))
            n_rows += 1
            assert rms <= rel_rms * float(b.std()), f"step {st['step']} {place}: rms of bf16 - fp32 {rms:.4f}"
            assert err <= tol, (f"step {st['step']} {place}: |bf16 - fp32| {err:.4f} > {tol:.4f} "
                                f"(entries {[(e['id'], len(e['tokens'])) for e in st['entries']]})")
            t16, t32 = int(np.argmax(a)), int(np.argmax(b))
            if t16 != t32:
                # another greedy token only where float32 itself has a near tie: within twice the bound
                assert b[t32] - b[t16] <= 2 * tol, (st["step"], place, t16, t32, b[t32] - b[t16], tol)
                flips.append((place, round(float(b[t32] - b[t16]) / float(b.std()), 4)))
    print(f"1.2B, 16 layers: {n_rows} rows, worst |bf16 - fp32| = {worst:.4f} of the logits' std (bound {rel:.4f}), "
          f"worst rms {worst_rms:.4f} (bound {rel_rms:.4f}); "
          f"{len(flips)} rows with another greedy token, all near ties: {flips[:8]}")
