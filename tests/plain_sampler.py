"""The reference's sampler restated in plain Python (float32 arithmetic where
the reference uses it), given the uniform number instead of a generator.

Order (src/sampler.c:334-352): repeat penalty -> greedy if temperature <= 0 or
top_k == 1 -> whole-vocabulary softmax if no filter is active -> else top-k (or
the 1024 largest), temperature softmax, top-p, min-p, inverse CDF."""
import numpy as np

TOP_FILTER_CAP = 1024          # src/sampler.c:7


def apply_repeat_penalty(logits, recent, last_n, penalty):
    """src/sampler.c:205-216: once per occurrence among the last n tokens."""
    out = np.array(logits, dtype=np.float32)
    if penalty == 1.0:
        return out
    for tok in list(recent)[max(0, len(recent) - last_n):]:
        if 0 <= tok < len(out):
            out[tok] = out[tok] / np.float32(penalty) if out[tok] > 0 else out[tok] * np.float32(penalty)
    return out


def argmax(logits):
    """src/sampler.c:125-136: the first maximum wins."""
    best, bestv = 0, logits[0]
    for i in range(1, len(logits)):
        if logits[i] > bestv:
            best, bestv = i, logits[i]
    return best


def sample(logits, u, temperature=0.8, top_k=40, top_p=0.9, min_p=0.1):
    """Returns (token, slack) where slack is how far ``u`` scaled by the sum is
    from the nearest CDF step (small slack: a neighbour is as right)."""
    l = np.asarray(logits, dtype=np.float32)
    V = len(l)
    f32 = np.float32
    if temperature <= 0 or top_k == 1:
        return argmax(l), np.inf
    inv_t = f32(1.0) / f32(temperature)
    if (top_k <= 0 or top_k >= V) and top_p >= 1.0 and min_p <= 0.0:
        # src/sampler.c:234-258
        mx = np.max(l * inv_t)
        e = np.exp((l * inv_t - mx).astype(np.float32)).astype(np.float32)
        cdf = np.cumsum(e.astype(np.float64))
        rnd = float(f32(u)) * cdf[-1]
        i = int(np.searchsorted(cdf, rnd, side="right"))
        i = min(i, V - 1)
        return i, float(np.min(np.abs(cdf - rnd)) / cdf[-1])
    k = top_k if 0 < top_k < V else min(V, TOP_FILTER_CAP)
    order = np.lexsort((np.arange(V), -l.astype(np.float64)))[:k]      # descending, lowest index first on ties
    vals = l[order]
    mx = vals[0] * inv_t
    ev = np.exp((vals * inv_t - mx).astype(np.float32)).astype(np.float32)
    s = f32(0)
    for x in ev:
        s = f32(s + x)
    kept = k
    if top_p < 1.0:                                                   # src/sampler.c:271-281
        cum = f32(0)
        for i in range(k):
            cum = f32(cum + f32(ev[i] / s))
            if cum > f32(top_p):
                kept = i + 1
                break
    if min_p > 0.0:                                                   # src/sampler.c:283-291
        min_prob = f32(f32(min_p) * f32(ev[0] / s))
        n = 0
        while n < kept and f32(ev[n] / s) >= min_prob:
            n += 1
        kept = n if n > 0 else 1
    psum = f32(0)
    for i in range(kept):
        psum = f32(psum + ev[i])
    rnd = f32(f32(u) * psum)
    acc, pick, slack = f32(0), kept - 1, np.inf
    for i in range(kept):                                             # src/sampler.c:293-310
        acc = f32(acc + ev[i])
        slack = min(slack, abs(float(acc) - float(rnd)) / float(psum))
        if rnd < acc:
            pick = i
            break
    return int(order[pick]), slack
