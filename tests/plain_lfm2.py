"""A plain, slow LFM2: whole sequences, no cache, one function for each part.

Written from the formulas of the reference (System64fumo/kappai; each function
cites the file and lines it restates).  It shares no code with the package: it
reads config.json and the safetensors file itself, with numpy only.  The
arithmetic runs in float64 by default so that it can judge the float32 path of
the engine as well as the bfloat16 one; ``dtype=np.float32`` gives the
reference's own precision.

``storage="bfloat16"`` makes it round to bfloat16 wherever the engine's bfloat16 mode stores a value in 16
bits (the normalised rows that feed a product, the outputs of in_proj / q,k,v / gate and up, the conv and
activation outputs, q and the cached k and v after the rotation, the softmax weights that go into the
product with V, the attention output), with everything else as exact as before: what an ideal
implementation with the engine's storage points computes.  The residual, the norms' statistics, the conv
sums, the softmax and the logits are never rounded.

Anchoring: tests/golden/ holds outputs of the reference's own C kernels
(compiled on the CPU from its source tree) for the parts below, and
tests/test_plain_vs_golden.py compares this file with them.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ----------------------------------------------------------------- file reading

def read_safetensors(path):
    """name -> numpy array (bfloat16 widened to float32, exactly)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        raw = data[b:en]
        if e["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
        elif e["dtype"] == "F32":
            a = np.frombuffer(raw, dtype=np.float32)
        elif e["dtype"] == "F16":
            a = np.frombuffer(raw, dtype=np.float16).astype(np.float32)
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = a.reshape(e["shape"]).copy()
    return out


def intermediate_size(cfg):
    """Width of the feed-forward from the config.json keys."""
    ff = cfg["block_ff_dim"]
    if cfg.get("block_auto_adjust_ff_dim", False):
        ff = (2 * ff) // 3
        if cfg.get("block_ffn_dim_multiplier") is not None:
            ff = int(cfg["block_ffn_dim_multiplier"] * ff)
        m = cfg.get("block_multiple_of", 256)
        ff = m * ((ff + m - 1) // m)
    return ff


def round_bf16(a):
    """Round to the nearest bfloat16 (ties to even), keeping the array's dtype."""
    a32 = np.ascontiguousarray(a, dtype=np.float32)
    u = a32.view(np.uint32)
    u = (u + (((u >> 16) & 1) + np.uint32(0x7FFF))) & np.uint32(0xFFFF0000)
    return u.view(np.float32).astype(a.dtype)


# ------------------------------------------------------------------------ parts

def embedding(table, tokens):
    """x[r,:] = E[tok[r],:], no scaling (src/backend/cpu/common.c:1774-1782; lfm2
    has no embedding scale, src/arch.c:73-82)."""
    return table[np.asarray(tokens, dtype=np.int64)]


def rmsnorm(x, w, eps):
    """y = x * (1/sqrt(mean(x^2) + eps)) * w over the last axis
    (src/backend/cpu/scalar/quants.c:1489-1512; per head :1521-1531)."""
    ss = np.sum(x * x, axis=-1, keepdims=True)
    scale = 1.0 / np.sqrt(ss / x.shape[-1] + eps)
    return (x * scale) * w


def linear(x, w, b=None):
    """y[n] = sum_k W[n,k] x[k], W row-major [out][in]
    (src/backend/cpu/scalar/quants.c:1367-1414)."""
    y = x @ w.T
    return y if b is None else y + b


def shortconv(p, conv_w, conv_b=None):
    """Gated causal depthwise convolution over one whole sequence from its
    start (src/backend/cpu/common.c:2393-2431): p = [B | C | X];
    bx_t = B_t * X_t; y_t = sum_k w[c,k] * bx_{t-(K-1)+k} (zero before the
    sequence; tap K-1 is the current token); out_t = C_t * y_t."""
    T, d3 = p.shape
    d = d3 // 3
    K = conv_w.shape[-1]
    w = conv_w.reshape(d, K)
    B, C, X = p[:, :d], p[:, d:2 * d], p[:, 2 * d:]
    bx = B * X
    padded = np.concatenate([np.zeros((K - 1, d), dtype=p.dtype), bx], axis=0)
    y = np.zeros((T, d), dtype=p.dtype)
    for k in range(K):
        y += padded[k:k + T] * w[:, k]
    if conv_b is not None:
        y = y + conv_b
    return C * y


def rope_tables(n_pos, rotary_dim, theta):
    """cos/sin of pos * theta^(-2j/rotary_dim), j < rotary_dim/2, in double
    (src/compute.c:22-65)."""
    half = rotary_dim // 2
    freq = np.power(float(theta), -2.0 * np.arange(half, dtype=np.float64) / rotary_dim)
    ang = np.arange(n_pos, dtype=np.float64)[:, None] * freq[None, :]
    return np.cos(ang), np.sin(ang)


def rope_neox(v, cos, sin):
    """v: [T, heads, hd]; pairs (j, j + half) (src/backend/cpu/quants.h:395-409)."""
    half = cos.shape[-1]
    a, b = v[..., :half], v[..., half:2 * half]
    c, s = cos[:, None, :], sin[:, None, :]
    out = v.copy()
    out[..., :half] = a * c - b * s
    out[..., half:2 * half] = a * s + b * c
    return out


def attention(q, k, v, scale, window=None, store=None):
    """Causal GQA attention of one whole sequence: q [T,H,hd], k,v [T,G,hd];
    head h reads kv head h // (H/G); keys 0..t (src/backend/cpu/scalar/core.c:
    383-433,623-666); scores = (q.k) * scale, softmax with the maximum
    subtracted, then sum p_t V_t."""
    T, H, hd = q.shape
    G = k.shape[1]
    rep = H // G
    out = np.zeros_like(q)
    for h in range(H):
        g = h // rep
        s = (q[:, h, :] @ k[:, g, :].T) * scale                     # [T, T]
        idx = np.arange(T)
        mask = idx[None, :] > idx[:, None]
        if window is not None:
            mask |= idx[None, :] < (idx[:, None] - window + 1)
        s = np.where(mask, -np.inf, s)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        if store is None:
            p = p / p.sum(axis=-1, keepdims=True)
            out[:, h, :] = p @ v[:, g, :]
        else:
            # the weights go into the product with V in 16 bits; their sum is taken before the rounding
            out[:, h, :] = (store(p) @ v[:, g, :]) / p.sum(axis=-1, keepdims=True)
    return out


def swiglu(g, u):
    """act = g / (1 + exp(-g)) * u (src/backend/cpu/scalar/core.c:774-800,
    src/backend/cpu/quants.h:369-371)."""
    return (g / (1.0 + np.exp(-g))) * u


# ------------------------------------------------------------------------ model

class PlainLfm2:
    def __init__(self, model_dir, dtype=np.float64, storage=None):
        with open(os.path.join(model_dir, "config.json")) as f:
            self.cfg = json.load(f)
        self.dtype = dtype
        if storage not in (None, "bfloat16"):
            raise ValueError("storage: None or 'bfloat16'")
        self.st = round_bf16 if storage == "bfloat16" else (lambda a: a)
        self.w = {k: v.astype(dtype) for k, v in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
        c = self.cfg
        self.d = c["hidden_size"]
        self.H = c["num_attention_heads"]
        self.G = c["num_key_value_heads"]
        self.hd = c.get("head_dim") or self.d // self.H
        self.eps = c["norm_eps"]
        self.theta = c.get("rope_theta", 1000000.0)
        self.ff = intermediate_size(c)
        self.bias = c.get("conv_bias", False)

    def conv_mixer(self, h, i):
        """src/models/lfm.c:7-21"""
        w, p = self.w, f"model.layers.{i}.conv."
        b = (lambda n: w[p + n + ".bias"]) if self.bias else (lambda n: None)
        proj = self.st(linear(h, w[p + "in_proj.weight"], b("in_proj")))
        y = self.st(shortconv(proj, w[p + "conv.weight"], b("conv")))
        return linear(y, w[p + "out_proj.weight"], b("out_proj"))

    def attention_mixer(self, h, i):
        """src/models/lfm.c:23-53"""
        w, p = self.w, f"model.layers.{i}.self_attn."
        T = h.shape[0]
        q = self.st(linear(h, w[p + "q_proj.weight"])).reshape(T, self.H, self.hd)
        k = self.st(linear(h, w[p + "k_proj.weight"])).reshape(T, self.G, self.hd)
        v = self.st(linear(h, w[p + "v_proj.weight"])).reshape(T, self.G, self.hd)
        q = rmsnorm(q, w[p + "q_layernorm.weight"], self.eps)
        k = rmsnorm(k, w[p + "k_layernorm.weight"], self.eps)
        cos, sin = rope_tables(T, self.hd, self.theta)
        q = self.st(rope_neox(q, cos.astype(self.dtype), sin.astype(self.dtype)))
        k = self.st(rope_neox(k, cos.astype(self.dtype), sin.astype(self.dtype)))
        rounded = self.st is round_bf16
        o = self.st(attention(q, k, v, 1.0 / math.sqrt(self.hd), store=round_bf16 if rounded else None))   # src/recipe/builders.c:244-248
        return linear(o.reshape(T, self.H * self.hd), w[p + "out_proj.weight"])

    def feed_forward(self, h, i):
        """src/recipe/builders.c:344-388"""
        w, p = self.w, f"model.layers.{i}.feed_forward."
        g, u = self.st(linear(h, w[p + "w1.weight"])), self.st(linear(h, w[p + "w3.weight"]))
        return linear(self.st(swiglu(g, u)), w[p + "w2.weight"])

    def hidden(self, tokens, trace=None):
        """The residual behind the last layer; ``trace`` (a list) gets a copy of it behind the embedding and
        behind every layer."""
        w = self.w
        x = embedding(w["model.embed_tokens.weight"], tokens)
        if trace is not None:
            trace.append(x.copy())
        for i, kind in enumerate(self.cfg["layer_types"]):
            p = f"model.layers.{i}."
            h = self.st(rmsnorm(x, w[p + "operator_norm.weight"], self.eps))
            x = x + (self.conv_mixer(h, i) if kind == "conv" else self.attention_mixer(h, i))
            h = self.st(rmsnorm(x, w[p + "ffn_norm.weight"], self.eps))
            x = x + self.feed_forward(h, i)
            if trace is not None:
                trace.append(x.copy())
        return x

    def logits(self, tokens):
        """[T, vocab] for the whole sequence (src/recipe/builders.c:450-468)."""
        x = self.hidden(tokens)
        h = self.st(rmsnorm(x, self.w["model.embedding_norm.weight"], self.eps))
        head = self.w["model.embed_tokens.weight"] if self.cfg.get("tie_embedding", True) else self.w["lm_head.weight"]
        return linear(h, head)
