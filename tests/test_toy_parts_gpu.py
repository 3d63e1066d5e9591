"""The framework's seams, shown with toy parts defined here and registered
from outside: a mixer with state of its own, a whole toy architecture built and
stepped through the engine with no change to the framework's files, and a
schedule that names a layer twice and lets a layer read another layer's cache."""
import json
import math
import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_lfm2 as P
from tolerances import tol_for

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------ a toy mixer
def make_toy():
    from kappai_b200.cache import StateSpec
    from kappai_b200.parts import Part, WeightSpec

    class EmaMixer(Part):
        """y_t = a * y_{t-1} + (1 - a) * h_t per channel (a = sigmoid(decay)), out = y W^T.
        State: y of the request's last token, zero at a sequence's start."""
        category = "mixer"

        def __init__(self, params, env):
            super().__init__(params, env)
            self.d = params["hidden_size"]

        def weight_specs(self):
            return {"decay": WeightSpec((self.d,), "bias"), "proj.weight": WeightSpec((self.d, self.d))}

        def bind(self, w):
            self.a = torch.sigmoid(w["decay"].float() * 50)
            self.w = w["proj.weight"].float()

        def cache_spec(self):
            return StateSpec((self.d,), "float32")

        def forward(self, h, residual, ctx, cache):
            h = h.float()
            for s in range(ctx.n_seg):
                r0, r1 = ctx.host_cu_rows[s], ctx.host_cu_rows[s + 1]
                slot = ctx.host_seg_slot[s]
                y = torch.zeros(self.d, device=h.device) if ctx.host_seg_pos[s] == 0 else cache.tensor[slot].clone()
                ys = []
                for r in range(r0, r1):
                    y = self.a * y + (1 - self.a) * h[r]
                    ys.append(y)
                cache.tensor[slot] = y
                residual[r0:r1] += torch.stack(ys) @ self.w.t()

    return EmaMixer


@dataclass
class _Unused:
    pass


def toy_config_cls():
    from kappai_b200.config import TypedConfig, cfg

    @dataclass
    class ToyConfig(TypedConfig):
        vocab_size: int = cfg()
        width: int = cfg()
        depth: int = cfg()
        ff: int = cfg()
        max_len: int = cfg(64)

    return ToyConfig


def toy_build_spec(c):
    from kappai_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    norm = lambda p: PartSpec("rmsnorm", {"size": c.width, "eps": 1e-5}, p)
    layers = [LayerSpec(mixer=PartSpec("toy_ema", {"hidden_size": c.width}, f"blocks.{i}.ema."),
                        ffn=PartSpec("swiglu", {"hidden_size": c.width, "intermediate_size": c.ff}, f"blocks.{i}.mlp."),
                        mixer_norm=norm(f"blocks.{i}.n1."), ffn_norm=norm(f"blocks.{i}.n2."))
              for i in range(c.depth)]
    return ModelSpec("ToyForCausalLM", c.width, c.vocab_size, c.max_len,
                     PartSpec("embedding", {"vocab_size": c.vocab_size, "hidden_size": c.width}, "emb."),
                     layers, [ScheduleEntry(i) for i in range(c.depth)], norm("final."),
                     PartSpec("lm_head", {"vocab_size": c.vocab_size, "hidden_size": c.width, "tied": True}, "head."))


def toy_plain_logits(w, cfg, toks):
    x = w["emb.weight"][np.asarray(toks)]
    for i in range(cfg["depth"]):
        p = f"blocks.{i}."
        h = P.rmsnorm(x, w[p + "n1.weight"], 1e-5)
        a = 1 / (1 + np.exp(-w[p + "ema.decay"] * 50))
        y, ys = np.zeros(cfg["width"]), []
        for t in range(len(toks)):
            y = a * y + (1 - a) * h[t]
            ys.append(y)
        x = x + np.stack(ys) @ w[p + "ema.proj.weight"].T
        h = P.rmsnorm(x, w[p + "n2.weight"], 1e-5)
        x = x + P.linear(P.swiglu(P.linear(h, w[p + "mlp.gate_proj.weight"]), P.linear(h, w[p + "mlp.up_proj.weight"])),
                         w[p + "mlp.down_proj.weight"])
    return P.linear(P.rmsnorm(x, w["final.weight"], 1e-5), w["emb.weight"])


def test_toy_architecture_with_a_stateful_mixer(tmp_path):
    from kappai_b200 import ModelRunner, StepEntry, write_random_model, Engine, EngineArgs, SamplingParams
    from kappai_b200.config import register_architecture, unregister_architecture
    from kappai_b200.parts import register_part, unregister_part
    register_part("mixer", "toy_ema", make_toy())
    register_architecture("ToyForCausalLM", toy_config_cls(), toy_build_spec)
    try:
        cfg = dict(architectures=["ToyForCausalLM"], vocab_size=97, width=24, depth=3, ff=40, max_len=64)
        d = write_random_model(cfg, str(tmp_path / "toy"), 4)
        w = {k: v.astype(np.float64) for k, v in P.read_safetensors(os.path.join(d, "model.safetensors")).items()}
        assert "blocks.2.ema.decay" in w and "blocks.0.mlp.gate_proj.weight" in w
        rng = np.random.default_rng(0)
        seqs = {"a": rng.integers(0, 97, 50).tolist(), "b": rng.integers(0, 97, 23).tolist()}
        ref = {k: toy_plain_logits(w, cfg, t) for k, t in seqs.items()}
        r = ModelRunner(d, dtype="float32", max_tokens=128, page_size=16)
        assert not r.cache.pools                          # no paged group at all: state slots only
        got = {"a": [], "b": []}
        fed = {"a": 0, "b": 0}
        plan = [{"a": 7}, {"a": 2, "b": 20}, {"a": 1, "b": 1}, {"b": 2}, {"a": 40}]
        for st in plan:
            ents = [StepEntry(k, seqs[k][fed[k]:fed[k] + n], list(range(n))) for k, n in st.items()]
            out = r.step(ents).cpu().double().numpy()
            o = 0
            for k, n in st.items():
                got[k].append(out[o:o + n]); o += n; fed[k] += n
        for k in seqs:
            assert np.abs(np.concatenate(got[k]) - ref[k]).max() < 1e-4, k
        r.end("a"); r.end("b")
        # and through the scheduler and sampler
        eng = Engine(EngineArgs(model=d, dtype="float32", max_batch=2, max_step_tokens=8, page_size=16, kv_tokens=128))
        outs = eng.generate([seqs["a"][:9], seqs["b"][:4]], SamplingParams(temperature=0.0, n_predict=5))
        for p, o in zip([seqs["a"][:9], seqs["b"][:4]], outs):
            seq = list(p)
            for t in o:
                lg = toy_plain_logits(w, cfg, seq)[-1]
                assert t == int(np.argmax(lg)) or lg.max() - lg[t] < 1e-4
                seq.append(t)
    finally:
        unregister_part("mixer", "toy_ema")
        unregister_architecture("ToyForCausalLM")


# ------------------------- a toy position encoding and a toy feed-forward with routing
def make_toy_position():
    from kappai_b200.parts import Part

    class LinearRotary(Part):
        """Pairs (2j, 2j+1) of the first ``n_rot`` dims of every head turn by ``pos * step * (j + 1)``."""
        category = "position"
        graph_safe = True                     # reads ctx.positions on the device only

        def __init__(self, params, env):
            super().__init__(params, env)
            self.n_rot, self.step, self.hd = params["n_rot"], params["step"], params["head_dim"]

        def apply(self, q, k, ctx):
            j = torch.arange(self.n_rot // 2, device=q.device, dtype=torch.float32)
            ang = ctx.positions.float()[:, None] * (self.step * (j + 1))[None, :]
            cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            for t in (q, k):
                v = t.unflatten(1, (-1, self.hd))
                x0, x1 = v[..., 0:self.n_rot:2].float().clone(), v[..., 1:self.n_rot:2].float().clone()
                v[..., 0:self.n_rot:2] = (x0 * cos - x1 * sin).to(t.dtype)
                v[..., 1:self.n_rot:2] = (x0 * sin + x1 * cos).to(t.dtype)

    return LinearRotary


def make_toy_experts():
    from kappai_b200.ops.linear import linear, linear_swiglu
    from kappai_b200.parts import Part, WeightSpec

    class Top1Experts(Part):
        """Router logits h R^T, softmax in float32, the best expert's SwiGLU output times its probability."""
        category = "feed_forward"

        def __init__(self, params, env):
            super().__init__(params, env)
            self.d, self.ff, self.E = params["hidden_size"], params["intermediate_size"], params["n_experts"]

        def weight_specs(self):
            s = {"router.weight": WeightSpec((self.E, self.d))}
            for e in range(self.E):
                s[f"experts.{e}.gate_proj.weight"] = WeightSpec((self.ff, self.d))
                s[f"experts.{e}.up_proj.weight"] = WeightSpec((self.ff, self.d))
                s[f"experts.{e}.down_proj.weight"] = WeightSpec((self.d, self.ff))
            return s

        def bind(self, w):
            self.router = (w["router.weight"] * 8).contiguous()          # (larger logits: clear choices)
            self.w_gu = [torch.cat([w[f"experts.{e}.gate_proj.weight"], w[f"experts.{e}.up_proj.weight"]], 0).contiguous()
                         for e in range(self.E)]
            self.w_down = [w[f"experts.{e}.down_proj.weight"].contiguous() for e in range(self.E)]

        def forward(self, h, residual, ctx):
            p = torch.softmax(linear(h, self.router, out_dtype=torch.float32), -1)
            gate, top = p.max(-1)
            for e in range(self.E):
                rows = (top == e).nonzero().flatten()
                if rows.numel():
                    y = linear(linear_swiglu(h[rows].contiguous(), self.w_gu[e]), self.w_down[e], out_dtype=torch.float32)
                    residual.index_add_(0, rows, y * gate[rows, None])

    return Top1Experts


def routed_config_cls():
    from kappai_b200.config import TypedConfig, cfg

    @dataclass
    class RoutedConfig(TypedConfig):
        vocab_size: int = cfg()
        width: int = cfg()
        depth: int = cfg()
        heads: int = cfg()
        kv_heads: int = cfg()
        head_dim: int = cfg()
        ff: int = cfg()
        n_experts: int = cfg()
        window: int = cfg()
        max_len: int = cfg(128)

    return RoutedConfig


def routed_build_spec(c):
    from kappai_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    norm = lambda p: PartSpec("rmsnorm", {"size": c.width, "eps": 1e-5}, p)
    pos = PartSpec("toy_linear_rotary", {"n_rot": c.head_dim // 2, "step": 0.05, "head_dim": c.head_dim})
    att = lambda i: PartSpec("attention", {"hidden_size": c.width, "num_heads": c.heads, "num_kv_heads": c.kv_heads,
                                           "head_dim": c.head_dim, "scale": c.head_dim ** -0.5,
                                           "window": c.window if i % 2 else None, "position": pos}, f"l.{i}.att.")
    layers = [LayerSpec(mixer=att(i),
                        ffn=PartSpec("toy_top1", {"hidden_size": c.width, "intermediate_size": c.ff,
                                                  "n_experts": c.n_experts}, f"l.{i}.moe."),
                        mixer_norm=norm(f"l.{i}.n1."), ffn_norm=norm(f"l.{i}.n2."))
              for i in range(c.depth)]
    return ModelSpec("RoutedToyForCausalLM", c.width, c.vocab_size, c.max_len,
                     PartSpec("embedding", {"vocab_size": c.vocab_size, "hidden_size": c.width}, "emb."),
                     layers, [ScheduleEntry(i) for i in range(c.depth)], norm("final."),
                     PartSpec("lm_head", {"vocab_size": c.vocab_size, "hidden_size": c.width, "tied": True}, "head."))


def routed_plain_logits(w, c, toks):
    T, H, G, hd = len(toks), c["heads"], c["kv_heads"], c["head_dim"]
    n_rot = hd // 2
    ang = np.arange(T)[:, None] * (0.05 * (np.arange(n_rot // 2) + 1))[None, :]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]

    def turn(v):
        v = v.copy()
        x0, x1 = v[..., 0:n_rot:2].copy(), v[..., 1:n_rot:2].copy()
        v[..., 0:n_rot:2], v[..., 1:n_rot:2] = x0 * cos - x1 * sin, x0 * sin + x1 * cos
        return v

    x = w["emb.weight"][np.asarray(toks)]
    for i in range(c["depth"]):
        p = f"l.{i}."
        h = P.rmsnorm(x, w[p + "n1.weight"], 1e-5)
        q = turn(P.linear(h, w[p + "att.q_proj.weight"]).reshape(T, H, hd))
        k = turn(P.linear(h, w[p + "att.k_proj.weight"]).reshape(T, G, hd))
        v = P.linear(h, w[p + "att.v_proj.weight"]).reshape(T, G, hd)
        o = P.attention(q, k, v, hd ** -0.5, c["window"] if i % 2 else None)
        x = x + P.linear(o.reshape(T, -1), w[p + "att.out_proj.weight"])
        h = P.rmsnorm(x, w[p + "n2.weight"], 1e-5)
        lg = P.linear(h, w[p + "moe.router.weight"] * 8)
        pr = np.exp(lg - lg.max(-1, keepdims=True))
        pr /= pr.sum(-1, keepdims=True)
        top = pr.argmax(-1)
        ranked = np.sort(pr, -1)
        assert (ranked[:, -1] - ranked[:, -2]).min() > 1e-4 and len(set(top.tolist())) > 1     # clear choices, several experts
        y = np.zeros_like(x)
        for t in range(T):
            e = f"{p}moe.experts.{top[t]}."
            f = P.swiglu(P.linear(h[t:t + 1], w[e + "gate_proj.weight"]), P.linear(h[t:t + 1], w[e + "up_proj.weight"]))
            y[t] = pr[t, top[t]] * P.linear(f, w[e + "down_proj.weight"])[0]
        x = x + y
    return P.linear(P.rmsnorm(x, w["final.weight"], 1e-5), w["emb.weight"])


def test_toy_architecture_with_its_own_position_encoding_and_routed_experts(tmp_path):
    """Attention (the framework's part and kernels, one layer with a window) with a position encoding defined
    here, and a feed-forward that routes every row to one of three experts, also defined here: registered,
    built from a configuration of its own, stepped in portions and decoded, against a plain computation."""
    from kappai_b200 import ModelRunner, StepEntry, write_random_model
    from kappai_b200.config import register_architecture, unregister_architecture
    from kappai_b200.parts import register_part, unregister_part
    register_part("position", "toy_linear_rotary", make_toy_position())
    register_part("feed_forward", "toy_top1", make_toy_experts())
    register_architecture("RoutedToyForCausalLM", routed_config_cls(), routed_build_spec)
    try:
        c = dict(architectures=["RoutedToyForCausalLM"], vocab_size=113, width=40, depth=3, heads=6, kv_heads=2,
                 head_dim=16, ff=24, n_experts=3, window=9, max_len=128)
        d = write_random_model(c, str(tmp_path / "routed"), 6)
        w = {k: v.astype(np.float64) for k, v in P.read_safetensors(os.path.join(d, "model.safetensors")).items()}
        rng = np.random.default_rng(2)
        seqs = {"a": rng.integers(0, 113, 70).tolist(), "b": rng.integers(0, 113, 31).tolist()}
        ref = {k: routed_plain_logits(w, c, t) for k, t in seqs.items()}
        r = ModelRunner(d, dtype="float32", max_tokens=128, page_size=16)
        assert len(r.cache.pools) == 2                     # layers that keep all keys, and the one with a window
        assert not r.model.graph_safe                      # the routed part is not: every step runs eagerly
        got, fed = {"a": [], "b": []}, {"a": 0, "b": 0}
        plan = [{"a": 30}, {"a": 2, "b": 29}, {"a": 1, "b": 1}, {"b": 1}, {"a": 37}]
        for st in plan:
            ents = [StepEntry(k, seqs[k][fed[k]:fed[k] + n], list(range(n))) for k, n in st.items()]
            out = r.step(ents).cpu().double().numpy()
            o = 0
            for k, n in st.items():
                got[k].append(out[o:o + n]); o += n; fed[k] += n
        for k in seqs:
            err = np.abs(np.concatenate(got[k]) - ref[k]).max()
            assert err <= tol_for("float32", ref[k]), (k, err)
        r.end("a"); r.end("b")
        r.cache.check()
    finally:
        unregister_part("position", "toy_linear_rotary")
        unregister_part("feed_forward", "toy_top1")
        unregister_architecture("RoutedToyForCausalLM")


# ----------------------------------- the schedule is data: twice, and a borrowed cache
def test_layer_named_twice_and_borrowed_cache(model_dirs, plain_models):
    """Schedule [0, 1, 2, 3, 1, 3*] over Tiny A's four layers: layer 1 (attention) runs twice with a
    cache of its own each time; the last entry runs layer 3 again but reads the keys and values that
    layer 3's first run cached (it computes only its own queries)."""
    from kappai_b200 import ModelRunner, StepEntry
    from kappai_b200.config import ScheduleEntry, register_architecture, unregister_architecture, lookup_architecture
    from kappai_b200.models.lfm2 import Lfm2Config, build_spec
    plain = plain_models["A"]

    def build(c):
        spec = build_spec(c)
        spec.architecture = "Lfm2Twice"
        spec.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(3), ScheduleEntry(1),
                         ScheduleEntry(3, cache_of=3)]
        return spec

    register_architecture("Lfm2Twice", Lfm2Config, build)
    try:
        d = model_dirs["A"]
        import shutil, tempfile
        d2 = tempfile.mkdtemp()
        shutil.copy(os.path.join(d, "model.safetensors"), d2)
        with open(os.path.join(d, "config.json")) as f:
            c = json.load(f)
        c["architectures"] = ["Lfm2Twice"]
        with open(os.path.join(d2, "config.json"), "w") as f:
            json.dump(c, f)
        rng = np.random.default_rng(1)
        toks = rng.integers(0, 256, 45).tolist()
        # plain: the same order by hand
        w, T = plain.w, len(toks)
        x = P.embedding(w["model.embed_tokens.weight"], toks)
        kv3 = {}

        def attn(h, i, borrowed=None):
            p = f"model.layers.{i}.self_attn."
            q = P.linear(h, w[p + "q_proj.weight"]).reshape(T, plain.H, plain.hd)
            q = P.rmsnorm(q, w[p + "q_layernorm.weight"], plain.eps)
            cos, sin = P.rope_tables(T, plain.hd, plain.theta)
            q = P.rope_neox(q, cos, sin)
            if borrowed is None:
                k = P.linear(h, w[p + "k_proj.weight"]).reshape(T, plain.G, plain.hd)
                v = P.linear(h, w[p + "v_proj.weight"]).reshape(T, plain.G, plain.hd)
                k = P.rope_neox(P.rmsnorm(k, w[p + "k_layernorm.weight"], plain.eps), cos, sin)
                kv3[i] = (k, v)
            else:
                k, v = borrowed
            o = P.attention(q, k, v, 1 / math.sqrt(plain.hd))
            return P.linear(o.reshape(T, -1), w[p + "out_proj.weight"])

        for i, borrow in [(0, None), (1, None), (2, None), (3, None), (1, None), (3, "yes")]:
            p = f"model.layers.{i}."
            h = P.rmsnorm(x, w[p + "operator_norm.weight"], plain.eps)
            if plain.cfg["layer_types"][i] == "conv":
                x = x + plain.conv_mixer(h, i)
            else:
                x = x + attn(h, i, kv3[3] if borrow else None)
            x = x + plain.feed_forward(P.rmsnorm(x, w[p + "ffn_norm.weight"], plain.eps), i)
        ref = P.linear(P.rmsnorm(x, w["model.embedding_norm.weight"], plain.eps), w["model.embed_tokens.weight"])
        for dtype in ("float32", "bfloat16"):
            r = ModelRunner(d2, dtype=dtype, max_tokens=128, page_size=16)
            assert r.storage.pools[next(iter(r.storage.pools))].shape[0] == 3       # entries 1, 3, 4 keep keys; 5 borrows
            got = []
            for a, b in [(0, 20), (20, 22), (22, 23), (23, 45)]:
                got.append(r.step([StepEntry("s", toks[a:b], list(range(b - a)))]).cpu().double().numpy())
            err = np.abs(np.concatenate(got) - ref).max()
            assert err <= tol_for(dtype, ref), (dtype, err)
    finally:
        unregister_architecture("Lfm2Twice")


# ------------------------- a toy mixer with a step table of its own, inside a captured decode step
def make_toy_with_table():
    from kappai_b200.cache import StateSpec
    from kappai_b200.engine.batch import PartTables
    from kappai_b200.parts import Part, WeightSpec

    class EmaTableMixer(Part):
        """The moving average of the first toy, but its decode steps read everything from device tensors: the
        host builds a table of its own for every step (``fresh``: 1 for a segment that starts its sequence,
        whose state counts as zero), which travels with the step's upload and, in a captured step, lives in the
        graph's static buffer."""
        category = "mixer"
        graph_safe = True
        step_tables_key = "toy_ema_fresh"
        calls = []                                     # (decode_only, fresh flags) of every table built: for the test

        def __init__(self, params, env):
            super().__init__(params, env)
            self.d = params["hidden_size"]

        def step_tables(self, segs):
            fresh = (np.asarray(segs.seg_pos) == 0).astype(np.int32)
            EmaTableMixer.calls.append((segs.decode_only, fresh.tolist()))
            return PartTables(arrays={"fresh": fresh}, scalars={"n": segs.n_seg})

        def weight_specs(self):
            return {"decay": WeightSpec((self.d,), "bias"), "proj.weight": WeightSpec((self.d, self.d))}

        def bind(self, w):
            self.a = torch.sigmoid(w["decay"].float() * 50)
            self.w = w["proj.weight"].float()

        def cache_spec(self):
            return StateSpec((self.d,), "float32")

        def forward(self, h, residual, ctx, cache):
            h = h.float()
            t = ctx.tables[self.step_tables_key]
            assert t.n == ctx.n_seg
            if ctx.decode_only:                         # device tensors only: can be captured
                slots = ctx.seg_slot.long()
                keep = (1 - t.fresh).float()[:, None]
                y = self.a * (cache.tensor[slots] * keep) + (1 - self.a) * h
                cache.tensor[slots] = y
                residual += y @ self.w.t()
                return
            for s in range(ctx.n_seg):
                r0, r1 = ctx.host_cu_rows[s], ctx.host_cu_rows[s + 1]
                slot = ctx.host_seg_slot[s]
                y = torch.zeros(self.d, device=h.device) if ctx.host_seg_pos[s] == 0 else cache.tensor[slot].clone()
                ys = []
                for r in range(r0, r1):
                    y = self.a * y + (1 - self.a) * h[r]
                    ys.append(y)
                cache.tensor[slot] = y
                residual[r0:r1] += torch.stack(ys) @ self.w.t()

    return EmaTableMixer


def test_a_part_with_a_step_table_of_its_own_runs_in_a_captured_step(tmp_path):
    from kappai_b200 import ModelRunner, StepEntry, write_random_model
    from kappai_b200.config import register_architecture, unregister_architecture
    from kappai_b200.parts import register_part, unregister_part
    Mixer = make_toy_with_table()
    register_part("mixer", "toy_ema", Mixer)
    register_architecture("ToyForCausalLM", toy_config_cls(), toy_build_spec)
    try:
        cfg = dict(architectures=["ToyForCausalLM"], vocab_size=97, width=24, depth=2, ff=40, max_len=64)
        d = write_random_model(cfg, str(tmp_path / "toy"), 6)
        w = {k: v.astype(np.float64) for k, v in P.read_safetensors(os.path.join(d, "model.safetensors")).items()}
        rng = np.random.default_rng(1)
        seqs = {"a": rng.integers(0, 97, 12).tolist(), "b": rng.integers(0, 97, 12).tolist()}
        ref = {k: toy_plain_logits(w, cfg, t) for k, t in seqs.items()}
        r = ModelRunner(d, dtype="float32", max_tokens=128, max_requests=2, page_size=16)
        assert r.model.graph_safe and list(r.model.table_builders) == ["toy_ema_fresh"]
        # "a" starts with a portion of 5 tokens (eager step); "b" token by token from its very first token, so
        # the first captured step has a fresh segment beside one that is not
        out = r.step([StepEntry("a", seqs["a"][:5], [4])]).cpu().double().numpy()
        assert np.abs(out[0] - ref["a"][4]).max() < 1e-4
        for i in range(7):
            ents = [StepEntry("a", [seqs["a"][5 + i]], [0]), StepEntry("b", [seqs["b"][i]], [0])]
            out = r.step(ents).cpu().double().numpy()
            assert np.abs(out[0] - ref["a"][5 + i]).max() < 1e-4, i
            assert np.abs(out[1] - ref["b"][i]).max() < 1e-4, i
        assert r.graphs.n_captures == 1 and r.graphs.n_replays >= 6
        decode_tables = [fresh for decode_only, fresh in Mixer.calls if decode_only and len(fresh) == 2]
        assert [0, 1] in decode_tables and decode_tables[-1] == [0, 0]        # the table was rebuilt for the replays
    finally:
        unregister_part("mixer", "toy_ema")
        unregister_architecture("ToyForCausalLM")
