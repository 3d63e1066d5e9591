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

Whole models too: the reference's loader, recipe builder, executor and CPU backend are compiled in place
(model.c includes a json-c header that this path never uses: a two-line stand-in is put on the include path;
the dozen symbols of the monitor, the safetensors reader and other parts that are not built are stubbed),
tiny LFM2 models with the package's random weights are written as GGUF files, and ref_model.c runs them
through ``compute_forward_batch`` whole, token by token and in portions.  The logits are saved; the test
compares the plain implementation's with them, which pins the order of a layer's operations, the mapping of
query heads to kv heads and the tensor names, not only the single kernels.

    python tests/golden/make_golden.py REF          (REF: a checkout of the reference; or $KAPPAI_REFERENCE)
"""
import ctypes
import glob
import os
import struct
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


# ------------------------------------------------------------------ whole models through the reference
MODEL_SOURCES = ["arch.c", "common.c", "compute.c", "config.c", "gguf.c", "kvcache.c", "log.c", "memory.c", "model.c",
                 "profile.c", "sampler.c", "threadpool.c", "weights.c", "cpu_topology.c", "hcs.c", "recipe/*.c",
                 "models/lfm.c", "models/llama.c", "backend/backend.c", "backend/cpu/common.c", "backend/cpu/nn_ops.c",
                 "backend/cpu/scalar/core.c", "backend/cpu/scalar/quants.c", "moe/*.c"]
DATA_SYMBOLS = {"g_monitor"}             # among the stubbed names, those that are variables


def build_model_lib(ref):
    tmp = tempfile.mkdtemp(prefix="golden_model_")
    shim = os.path.join(tmp, "shim", "json-c")
    os.makedirs(shim)
    for h in ("json.h", "json_types.h"):
        with open(os.path.join(shim, h), "w") as f:
            f.write("#pragma once\ntypedef struct json_object json_object;\ntypedef struct json_tokener json_tokener;\n")
    src = os.path.join(ref, "src")
    files = [os.path.join(HERE, "ref_model.c")]
    for pat in MODEL_SOURCES:
        files += sorted(glob.glob(os.path.join(src, pat)))
    base = ["gcc", "-std=gnu11", "-O1", "-fPIC", "-w", "-I", os.path.join(tmp, "shim"), "-I", src]
    objs = []
    for i, f in enumerate(files):
        o = os.path.join(tmp, f"o{i}.o")
        subprocess.run(base + ["-c", f, "-o", o], check=True)
        objs.append(o)
    first = os.path.join(tmp, "first.so")
    subprocess.run(["gcc", "-shared", "-o", first] + objs + ["-lm", "-lpthread"], check=True)
    und = subprocess.run(["nm", "-u", "--dynamic", first], capture_output=True, text=True, check=True).stdout
    names = [l.split()[1] for l in und.splitlines() if len(l.split()) == 2 and l.split()[0] == "U" and "@" not in l]
    stubs = os.path.join(tmp, "stubs.c")
    with open(stubs, "w") as f:
        f.write("/* symbols of parts of the reference that are not built here and that these runs never reach */\n")
        for n in names:
            f.write(f"void *{n} = 0;\n" if n in DATA_SYMBOLS else f"long {n}(void) {{ return 0; }}\n")
    lib = os.path.join(tmp, "libgoldenmodel.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-w", "-o", lib, stubs] + objs + ["-lm", "-lpthread"], check=True)
    return ctypes.CDLL(lib), names


def _gguf_string(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, cfg, w, ff):
    """An LFM2 model as a GGUF file of float32 tensors, with the keys and names of the reference's own test
    writer (src/test/test_synth_gguf.c:349-460).  ``w``: tensor name of the model folder -> array."""
    d, H, G = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    kv = []
    k_str = lambda k, v: kv.append(_gguf_string(k) + struct.pack("<I", 8) + _gguf_string(v))
    k_i32 = lambda k, v: kv.append(_gguf_string(k) + struct.pack("<Ii", 5, v))
    k_f32 = lambda k, v: kv.append(_gguf_string(k) + struct.pack("<If", 6, v))
    k_str("general.architecture", "lfm2")
    k_i32("lfm2.context_length", cfg["max_position_embeddings"])
    k_i32("lfm2.block_count", cfg["num_hidden_layers"])
    k_i32("lfm2.embedding_length", d)
    k_i32("lfm2.feed_forward_length", ff)
    k_i32("lfm2.attention.head_count", H)
    heads_kv = [0 if t == "conv" else G for t in cfg["layer_types"]]
    kv.append(_gguf_string("lfm2.attention.head_count_kv") + struct.pack("<IIQ", 9, 5, len(heads_kv))
              + struct.pack(f"<{len(heads_kv)}i", *heads_kv))
    k_i32("lfm2.attention.key_length", cfg.get("head_dim") or d // H)
    k_f32("lfm2.attention.layer_norm_rms_epsilon", cfg["norm_eps"])
    k_i32("lfm2.shortconv.l_cache", cfg["conv_L_cache"])
    k_f32("lfm2.rope.freq_base", cfg["rope_theta"])
    tensors = []
    add = lambda name, a: tensors.append((name, np.ascontiguousarray(a, dtype=np.float32)))
    add("token_embd.weight", w["model.embed_tokens.weight"])
    add("output_norm.weight", w["model.embedding_norm.weight"])
    if not cfg.get("tie_embedding", True):
        add("output.weight", w["lm_head.weight"])
    for i, t in enumerate(cfg["layer_types"]):
        p = f"model.layers.{i}."
        add(f"blk.{i}.attn_norm.weight", w[p + "operator_norm.weight"])
        if t == "conv":
            add(f"blk.{i}.shortconv.in_proj.weight", w[p + "conv.in_proj.weight"])
            add(f"blk.{i}.shortconv.conv.weight", w[p + "conv.conv.weight"].reshape(d, -1))
            add(f"blk.{i}.shortconv.out_proj.weight", w[p + "conv.out_proj.weight"])
        else:
            for a, b in (("attn_q", "q_proj"), ("attn_k", "k_proj"), ("attn_v", "v_proj"), ("attn_output", "out_proj")):
                add(f"blk.{i}.{a}.weight", w[p + f"self_attn.{b}.weight"])
            add(f"blk.{i}.attn_q_norm.weight", w[p + "self_attn.q_layernorm.weight"])
            add(f"blk.{i}.attn_k_norm.weight", w[p + "self_attn.k_layernorm.weight"])
        add(f"blk.{i}.ffn_norm.weight", w[p + "ffn_norm.weight"])
        add(f"blk.{i}.ffn_gate.weight", w[p + "feed_forward.w1.weight"])
        add(f"blk.{i}.ffn_up.weight", w[p + "feed_forward.w3.weight"])
        add(f"blk.{i}.ffn_down.weight", w[p + "feed_forward.w2.weight"])
    infos, off = [], 0
    for name, a in tensors:
        dims = list(reversed(a.shape))                               # GGUF dims are fastest first
        infos.append(_gguf_string(name) + struct.pack("<I", len(dims)) + struct.pack(f"<{len(dims)}Q", *dims)
                     + struct.pack("<IQ", 0, off))
        off += (a.nbytes + 31) // 32 * 32
    head = struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(kv)) + b"".join(kv) + b"".join(infos)
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * ((-len(head)) % 32))
        for name, a in tensors:
            f.write(a.tobytes())
            f.write(b"\0" * ((-a.nbytes) % 32))


# Models that the reference's LFM2 can run: no biases (it has none), and head_dim = hidden / heads as in every
# real LFM2 file (with another head size the reference's conv layers write their rows with the stride of the
# attention buffer, src/recipe/ops_hybrid.c:335-336, which the product that follows does not expect: its
# results for several rows at once are then not those of its own formulas).  Everything else as the tiny
# configurations.  tests/test_plain_vs_golden.py has the same table.
MODEL_CASES = {"A": {}, "B": {"conv_bias": False}, "C": {"hidden_size": 240}}
MODEL_CUTS = {"whole": lambda n: [0, n], "each": lambda n: list(range(n + 1)),
              "portions": lambda n: [c for c in (0, 7, 9, 25, 28, 30, 47, 49) if c < n] + [n]}


def model_cases(ref, out):
    root = os.path.dirname(os.path.dirname(HERE))
    for p in (root, os.path.join(root, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from kappai_b200.weights import write_random_model
    from plain_lfm2 import intermediate_size, read_safetensors
    from tiny_configs import CONFIGS

    lib, stubbed = build_model_lib(ref)
    out["model_stubbed"] = np.array(sorted(stubbed))
    for name, override in MODEL_CASES.items():
        cfg, seed = CONFIGS[name]
        cfg = dict(cfg, **override)
        d = tempfile.mkdtemp(prefix=f"golden_{name}_")
        write_random_model(cfg, d, seed)
        gg = os.path.join(d, "model.gguf")
        write_gguf(gg, cfg, read_safetensors(os.path.join(d, "model.safetensors")), intermediate_size(cfg))
        V = cfg["vocab_size"]
        toks = np.random.default_rng(100 + seed).integers(0, V, 61).astype(np.int32)
        out[f"model{name}_tokens"] = toks
        for cut_name, make in MODEL_CUTS.items():
            cuts = np.asarray(make(len(toks)), dtype=np.int32)
            rows = np.zeros((len(cuts) - 1, V), np.float32)
            rc = lib.gold_model_logits(gg.encode(), toks.ctypes.data_as(ctypes.c_void_p), cuts.ctypes.data_as(ctypes.c_void_p),
                                       len(cuts) - 1, cfg["max_position_embeddings"], 1, rows.ctypes.data_as(ctypes.c_void_p), V)
            if rc != 0:
                sys.exit(f"the reference failed on model {name}, cut '{cut_name}': {rc}")
            keep = np.arange(len(cuts) - 1) if len(cuts) <= 12 else np.array([0, 1, 2, 7, 15, 31, 32, len(cuts) - 2])
            out[f"model{name}_{cut_name}_positions"] = cuts[1:][keep] - 1       # the position whose logits a row holds
            out[f"model{name}_{cut_name}_logits"] = rows[keep]


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
    model_cases(ref, out)
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print(f"wrote {os.path.join(HERE, 'golden.npz')} with {len(out)} arrays")


if __name__ == "__main__":
    main()
