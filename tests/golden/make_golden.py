#!/usr/bin/env python3
"""Make tests/golden/golden.npz from the reference's own C kernels.

The reference (System64fumo/kappai) cannot be linked as shipped here (its
loader needs json-c), but its CPU kernels compile on their own.  This script
compiles four small harness files that ``#include`` the reference's sources in
place from REF/src (nothing is copied), stubs the symbols those files mention
but these cases never reach, and runs seeded cases through: rmsnorm,
rmsnorm_per_head, the rope table and NeoX rotation, the gated short convolution
with state, attention over its fp16 cache (online-softmax and plain), SwiGLU,
argmax and the sampler.  Inputs and outputs are saved; the test
tests/test_plain_vs_golden.py compares the plain implementation with them.

    python tests/golden/make_golden.py REF          (REF: a checkout of the reference; or $KAPPAI_REFERENCE)
"""
import ctypes
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
TUS = ["ref_core.c", "ref_common.c", "ref_misc.c", "ref_rope.c"]


def build(ref):
    tmp = tempfile.mkdtemp(prefix="golden_")
    srcs = [os.path.join(HERE, t) for t in TUS] + [os.path.join(ref, "src", "common.c")]
    base = ["gcc", "-std=gnu11", "-O1", "-fPIC", "-shared", "-w", "-I", os.path.join(ref, "src")]
    first = os.path.join(tmp, "first.so")
    subprocess.run(base + ["-o", first] + srcs + ["-lm"], check=True)
    und = subprocess.run(["nm", "-u", "--dynamic", first], capture_output=True, text=True, check=True).stdout
    names = [l.split()[1] for l in und.splitlines() if len(l.split()) == 2 and l.split()[0] == "U" and "@" not in l]
    stubs = os.path.join(tmp, "stubs.c")
    with open(stubs, "w") as f:
        f.write("/* symbols the included files mention but the golden cases never reach */\n")
        for n in names:
            f.write(f"long {n}(void) {{ return 0; }}\n")
    lib = os.path.join(tmp, "libgolden.so")
    subprocess.run(base + ["-o", lib] + srcs + [stubs, "-lm"], check=True)
    return ctypes.CDLL(lib)


def fp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("KAPPAI_REFERENCE")
    if not ref:
        sys.exit("usage: make_golden.py REF   (a checkout of the reference)")
    lib = build(ref)
    rng = np.random.default_rng(1234)
    f32 = lambda *s: rng.standard_normal(s).astype(np.float32)
    out = {}

    # rmsnorm and per-head rmsnorm
    for i, (n, eps) in enumerate([(64, 1e-5), (100, 1e-6), (7, 1e-5)]):
        x, w = f32(n) * 3, (1 + 0.1 * f32(n))
        y = np.zeros(n, np.float32)
        lib.gold_rmsnorm(fp(x), fp(w), fp(y), n, ctypes.c_float(eps))
        out[f"rmsnorm{i}_x"], out[f"rmsnorm{i}_w"], out[f"rmsnorm{i}_eps"], out[f"rmsnorm{i}_y"] = x, w, np.float64(eps), y
    x, w = f32(3 * 16), 1 + 0.1 * f32(16)
    y = np.zeros_like(x)
    lib.gold_rmsnorm_per_head(fp(x), fp(w), fp(y), 3, 16, ctypes.c_float(1e-5))
    out["perhead_x"], out["perhead_w"], out["perhead_y"] = x, w, y

    # rope table and rotation
    for i, (n_ctx, hd, theta) in enumerate([(300, 16, 1e4), (5000, 64, 1e6)]):
        c, s = np.zeros((n_ctx, hd // 2), np.float32), np.zeros((n_ctx, hd // 2), np.float32)
        lib.gold_rope_table(fp(c), fp(s), n_ctx, hd, ctypes.c_float(theta))
        keep = np.array(sorted(set([0, 1, 2, 100, n_ctx - 3, n_ctx - 1]) | {p for p in (4095, 4096, 4097) if p < n_ctx}))
        out[f"rope{i}_positions"], out[f"rope{i}_theta"] = keep, np.float64(theta)   # the table has a block edge at 4096
        out[f"rope{i}_cos"], out[f"rope{i}_sin"] = c[keep], s[keep]
        v = f32(3, hd)
        v2 = v.copy()
        pos = n_ctx - 3
        lib.gold_rope_neox(fp(v2), 3, hd, hd, fp(np.ascontiguousarray(c[pos])), fp(np.ascontiguousarray(s[pos])))
        out[f"rope{i}_v"], out[f"rope{i}_pos"], out[f"rope{i}_rot"] = v, np.int64(pos), v2

    # gated short convolution with state, in two chunks
    for i, (K, dim, r1, r2) in enumerate([(3, 7, 9, 4), (4, 5, 2, 6), (2, 6, 1, 1), (4, 3, 1, 2)]):
        mixed = f32(r1 + r2, 3 * dim)
        w = rng.uniform(-0.5, 0.5, (dim, K)).astype(np.float32)
        state = np.zeros((dim, K - 1), np.float32)          # the reference keeps [dim][K-1]
        o = np.zeros((r1 + r2, dim), np.float32)
        lib.gold_shortconv(fp(mixed), fp(w), fp(state), fp(o), r1, dim, K)
        mid = state.copy()
        lib.gold_shortconv(fp(np.ascontiguousarray(mixed[r1:])), fp(w), fp(state), fp(o[r1:]), r2, dim, K)
        out[f"conv{i}_mixed"], out[f"conv{i}_w"], out[f"conv{i}_out"] = mixed, w, o
        out[f"conv{i}_r1"], out[f"conv{i}_mid"], out[f"conv{i}_state"] = np.int64(r1), mid, state

    # attention of one query over n_pos cached keys (fp16 cache), both ways
    for i, (hd, n_pos) in enumerate([(16, 1), (16, 5), (16, 70), (64, 33)]):
        k, v, q = f32(n_pos, hd), f32(n_pos, hd), f32(hd)
        kr, vr = np.zeros_like(k), np.zeros_like(v)
        lib.gold_f16_round(fp(k), fp(kr), k.size)
        lib.gold_f16_round(fp(v), fp(vr), v.size)
        scale = 1.0 / np.sqrt(hd)
        for flash in (1, 0):
            o = np.zeros(hd, np.float32)
            lib.gold_attention(fp(k), fp(v), fp(q), fp(o), hd, n_pos, ctypes.c_float(scale), flash)
            out[f"attn{i}_out{flash}"] = o
        out[f"attn{i}_k16"], out[f"attn{i}_v16"], out[f"attn{i}_q"] = kr, vr, q

    # SwiGLU
    g, u = f32(3, 11) * 4, f32(3, 11)
    o = np.zeros_like(g)
    lib.gold_swiglu(fp(g), fp(u), fp(o), 11, 3)
    out["swiglu_g"], out["swiglu_u"], out["swiglu_o"] = g, u, o

    # argmax ties and the sampler
    l = f32(50)
    l[[7, 31]] = 9.0
    out["argmax_l"], out["argmax_i"] = l, np.int64(lib.gold_argmax(fp(l), 50))
    cases = [(0.8, 40, 0.9, 0.1), (1.3, 0, 1.0, 0.0), (0.5, 0, 0.7, 0.0), (1.0, 0, 1.0, 0.05), (0.8, 5, 1.0, 0.0),
             (2.0, 1000, 0.95, 0.0), (0.0, 40, 0.9, 0.1), (0.7, 1, 0.9, 0.1)]
    rows = []
    logits = (f32(len(cases) * 6, 300) * 3).astype(np.float16).astype(np.float32)   # fp16-exact: stores small
    for j in range(logits.shape[0]):
        t, k, p, m = cases[j % len(cases)]
        u = ctypes.c_float(0)
        seed = 1000 + j
        tok = lib.gold_sample(fp(np.ascontiguousarray(logits[j])), 300, ctypes.c_ulonglong(seed), ctypes.c_float(t), k,
                              ctypes.c_float(p), ctypes.c_float(m), ctypes.byref(u))
        rows.append((t, k, p, m, u.value, tok))
    out["sample_logits"], out["sample_rows"] = logits.astype(np.float16).astype(np.float32), np.array(rows, dtype=np.float64)

    out["sample_logits"] = out["sample_logits"].astype(np.float16)
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print(f"wrote {os.path.join(HERE, 'golden.npz')} with {len(out)} arrays")


if __name__ == "__main__":
    main()
