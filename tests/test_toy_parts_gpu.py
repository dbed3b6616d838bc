"""Generality of the parts: a toy mixer with state of its own, defined here, is registered,
built into a model beside an attention layer, loaded with random weights and stepped through
the engine, portions and mixed batches included, without any change to the package."""
from dataclasses import dataclass
from typing import ClassVar

import pytest
import torch

from helpers import random_ids

pytestmark = pytest.mark.gpu


def _register():
    from tinyserve_b200.config import (LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec,
                                       register_architecture)
    from tinyserve_b200.parts import Mixer, ParamSpec, StateSpec, register_mixer

    class DecayMixer(Mixer):
        """s_t = decay * s_{t-1} + x_t per request; out_t = s_t @ W^T.  The state s lives in
        the request's state slot between steps."""
        tree_name = "decay"

        def __init__(self, hidden_size, decay):
            super().__init__()
            self.hidden_size, self.decay = hidden_size, decay

        def param_specs(self):
            return {"proj.weight": ParamSpec((self.hidden_size, self.hidden_size))}

        def state_spec(self):
            return StateSpec((self.hidden_size,), "float32")

        def forward(self, h, ctx, call):
            state = ctx.state(call.state)
            cu, slots, fresh = ctx.host["cu_q"], ctx.host["state_slots"], ctx.host["fresh"]
            out = torch.empty_like(h, dtype=torch.float32)
            for b in range(ctx.num_requests):
                s = torch.zeros_like(state[slots[b]]) if fresh[b] else state[slots[b]].clone()
                for t in range(cu[b], cu[b + 1]):
                    s = self.decay * s + h[t].float()
                    out[t] = s
                if cu[b + 1] > cu[b]:
                    state[slots[b]] = s
            return (out @ self.w["proj.weight"].float().T).to(h.dtype)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyDecayForCausalLM"
        vocab_size: int = 0
        hidden_size: int = 0
        decay: float = 0.5
        heads: int = 2

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["vocab_size"], raw["hidden_size"], raw["decay"], raw["heads"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size,
                    "hidden_size": self.hidden_size, "decay": self.decay, "heads": self.heads}

        def model_spec(self):
            h = self.hidden_size
            norm = PartSpec("rmsnorm", {"eps": 1e-5})
            ffn = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": 2 * h, "activation": "gelu_tanh"})
            toy = LayerSpec(PartSpec("toy_decay", {"hidden_size": h, "decay": self.decay}), ffn, norm)
            attn = LayerSpec(PartSpec("attention", {
                "hidden_size": h, "num_heads": self.heads, "num_kv_heads": 1, "head_dim": 16,
                "position": PartSpec("rotary", {"rotary_dim": 8, "theta": 100.0, "pairing": "interleaved"})}),
                ffn, norm)
            # the toy layer runs twice (two states), the attention layer between them
            order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2))
            return ModelSpec(self.vocab_size, h, (toy, attn), order, norm, True)

    register_mixer("toy_decay", DecayMixer)
    register_architecture(ToyConfig.architecture, ToyConfig)
    return ToyConfig


def _plain_toy(weights, cfg, ids):
    """The toy model on a whole sequence, float64, written out by hand."""
    w = {k: v.double() for k, v in weights.items()}
    h = cfg.hidden_size
    norm = lambda x, wt: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * wt
    r = w["model.embed_tokens.weight"][torch.tensor(ids)]
    T = len(ids)

    def ffn(x, p):
        g, u = x @ w[p + "gate_proj.weight"].T, x @ w[p + "up_proj.weight"].T
        return (torch.nn.functional.gelu(g, approximate="tanh") * u) @ w[p + "down_proj.weight"].T

    def decay_mixer(x, p):
        s, out = torch.zeros(h, dtype=torch.float64), []
        for t in range(T):
            s = cfg.decay * s + x[t]
            out.append(s)
        return torch.stack(out) @ w[p + "proj.weight"].T

    def attention(x, p):
        H, D, R = cfg.heads, 16, 8
        q = (x @ w[p + "q_proj.weight"].T).view(T, H, D)
        k = (x @ w[p + "k_proj.weight"].T).view(T, 1, D)
        v = (x @ w[p + "v_proj.weight"].T).view(T, 1, D)
        inv = 1.0 / 100.0 ** (torch.arange(0, R, 2, dtype=torch.float64) / R)
        ang = torch.outer(torch.arange(T, dtype=torch.float64), inv)
        c, s = ang.cos().float().double()[:, None], ang.sin().float().double()[:, None]

        def rope(z):
            a, b = z[..., 0:R:2], z[..., 1:R:2]
            rot = torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2)
            return torch.cat([rot, z[..., R:]], -1)
        q, k = rope(q), rope(k)
        sc = torch.einsum("thd,sd->hts", q, k[:, 0]) * D ** -0.5
        mask = torch.arange(T)[None] <= torch.arange(T)[:, None]
        sc = sc.masked_fill(~mask[None], float("-inf"))
        o = torch.einsum("hts,sd->thd", sc.softmax(-1), v[:, 0]).reshape(T, H * D)
        return o @ w[p + "o_proj.weight"].T

    for layer, kind in ((0, "decay"), (1, "attn"), (0, "decay")):
        p = f"model.layers.{layer}."
        x = norm(r, w[p + "input_layernorm.weight"])
        r = r + (decay_mixer(x, p + "decay.") if kind == "decay" else attention(x, p + "self_attn."))
        r = r + ffn(norm(r, w[p + "post_attention_layernorm.weight"]), p + "mlp.")
    return norm(r, w["model.norm.weight"]) @ w["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 3e-2)])
def test_toy_mixer_with_state_runs_through_the_engine(dtype, tol, tmp_path):
    import os
    from safetensors.torch import load_file
    from tinyserve_b200.config import ARCHITECTURES, EngineConfig
    from tinyserve_b200.engine.batch import StepEntry
    from tinyserve_b200.engine.runner import ModelRunner
    from tinyserve_b200.parts.base import MIXERS
    from tinyserve_b200.weights import write_random_model
    ToyConfig = _register()
    try:
        cfg = ToyConfig(vocab_size=97, hidden_size=40, decay=0.7, heads=3)
        folder = write_random_model(cfg, str(tmp_path), seed=3)
        weights = load_file(os.path.join(folder, "model.safetensors"))
        assert "model.layers.0.decay.proj.weight" in weights
        runner = ModelRunner(EngineConfig(model=folder, dtype=dtype, max_model_len=128, block_size=8,
                                          max_num_seqs=3, max_num_batched_tokens=64, num_blocks=24))
        assert len(runner.model.state_entries) == 2 and runner.model.group_sizes == [1]
        assert runner.device_cache.states[0].shape == (3, 40)
        a, b = random_ids(97, 50, seed=1), random_ids(97, 23, seed=2)
        ref_a, ref_b = _plain_toy(weights, cfg, a), _plain_toy(weights, cfg, b)
        mgr = runner.manager
        mgr.begin("a"); mgr.begin("b")
        got_a, got_b = [], []
        # a in portions; b joins later, decodes beside a's portions; slots are used again after
        got_a.append(runner.step([StepEntry("a", a[:17], list(range(17)))]))
        out = runner.step([StepEntry("a", a[17:19], [0, 1]), StepEntry("b", b[:20], list(range(20)))])
        got_a.append(out[:2]); got_b.append(out[2:])
        for t in range(20, 23):
            out = runner.step([StepEntry("b", [b[t]], [0]), StepEntry("a", a[19 + (t - 20) * 9:28 + (t - 20) * 9], list(range(9)))])
            got_b.append(out[:1]); got_a.append(out[1:])
        got_a.append(runner.step([StepEntry("a", a[46:], list(range(4)))]))
        mgr.free("a"); mgr.free("b")
        for got, ref in ((torch.cat(got_a), ref_a), (torch.cat(got_b), ref_b)):
            assert (got.double().cpu() - ref).abs().max().item() < tol * ref.abs().max().item()
        # a new request in a used slot starts from a zero state
        mgr.begin("c")
        out = runner.step([StepEntry("c", b, list(range(23)))])
        assert (out.double().cpu() - ref_b).abs().max().item() < tol * ref_b.abs().max().item()
        mgr.free("c")
        mgr.check_invariants()
    finally:
        ARCHITECTURES.pop("ToyDecayForCausalLM", None)
        MIXERS.pop("toy_decay", None)


# ----------------------------------------------------------------------------- routing, positions
def _register_routed():
    """A toy feed-forward with top-1 routing over small experts (router logits in 32-bit) and a
    toy position encoding (rotary tables with linearly spaced frequencies and a position scale),
    both defined here, beside the package's attention."""
    from tinyserve_b200.config import (LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec,
                                       register_architecture)
    from tinyserve_b200.kernels import ops
    from tinyserve_b200.parts import FeedForward, ParamSpec
    from tinyserve_b200.parts.base import PositionEncoding, register_feed_forward, register_position_encoding

    class RoutedFFN(FeedForward):
        """y_t = down_e(gelu(up_e(x_t))) * p_e with e = argmax of the router's 32-bit logits and
        p_e its softmax probability: routing by data, experts as stacked tensors."""
        tree_name = "moe"

        def __init__(self, hidden_size, expert_size, num_experts):
            super().__init__()
            self.h, self.i, self.e = hidden_size, expert_size, num_experts

        def param_specs(self):
            return {"router.weight": ParamSpec((self.e, self.h)),
                    "up.weight": ParamSpec((self.e * self.i, self.h)),
                    "down.weight": ParamSpec((self.e * self.h, self.i))}

        def forward(self, h, ctx):
            logits = h.float() @ self.w["router.weight"].float().T
            prob, expert = logits.softmax(-1).max(-1)
            up = self.w["up.weight"].view(self.e, self.i, self.h)
            down = self.w["down.weight"].view(self.e, self.h, self.i)
            out = torch.zeros_like(h)
            for e in expert.unique().tolist():
                rows = (expert == e).nonzero().squeeze(-1)
                mid = torch.nn.functional.gelu(ops.materialize(ops.linear(h[rows].contiguous(), up[e])).float(),
                                               approximate="tanh").to(h.dtype)
                y = ops.materialize(ops.linear(mid, down[e]))
                out[rows] = (y.float() * prob[rows, None]).to(h.dtype)
            return out

    class LinearRotary(PositionEncoding):
        """Rotary tables with frequencies 1 / (1 + k) and positions divided by ``scale``: the
        attention part and its kernels only see rotary_dim, the pairing and the two tables."""

        def __init__(self, rotary_dim, scale):
            super().__init__()
            self.rotary_dim, self.scale, self.interleaved = rotary_dim, float(scale), False
            self.cos = self.sin = None

        def prepare(self, runtime):
            freq = 1.0 / (1.0 + torch.arange(self.rotary_dim // 2, dtype=torch.float64))
            ang = torch.outer(torch.arange(runtime.max_positions, dtype=torch.float64) / self.scale, freq)
            self.cos, self.sin = ang.cos().float().to(runtime.device), ang.sin().float().to(runtime.device)

    @dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyRoutedForCausalLM"
        vocab_size: int = 0
        hidden_size: int = 0
        experts: int = 0

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["vocab_size"], raw["hidden_size"], raw["experts"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size,
                    "hidden_size": self.hidden_size, "experts": self.experts}

        def model_spec(self):
            h = self.hidden_size
            norm = PartSpec("rmsnorm", {"eps": 1e-6})
            attn = PartSpec("attention", {
                "hidden_size": h, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                "position": PartSpec("toy_linear_rotary", {"rotary_dim": 16, "scale": 2.0})})
            routed = PartSpec("toy_routed", {"hidden_size": h, "expert_size": 24, "num_experts": self.experts})
            dense = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": 64, "activation": "silu"})
            layers = (LayerSpec(attn, routed, norm), LayerSpec(attn, dense, norm))
            return ModelSpec(self.vocab_size, h, layers, (LayerCall(0, 0), LayerCall(1, 1)), norm, False)

    register_feed_forward("toy_routed", RoutedFFN)
    register_position_encoding("toy_linear_rotary", LinearRotary)
    register_architecture(RoutedConfig.architecture, RoutedConfig)
    return RoutedConfig


def _plain_routed(weights, cfg, ids):
    w = {k: v.double() for k, v in weights.items()}
    T, h, H, Hkv, D = len(ids), cfg.hidden_size, 4, 2, 16
    norm = lambda x, wt: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * wt
    r = w["model.embed_tokens.weight"][torch.tensor(ids)]
    freq = 1.0 / (1.0 + torch.arange(D // 2, dtype=torch.float64))
    ang = torch.outer(torch.arange(T, dtype=torch.float64) / 2.0, freq)
    c, s = ang.cos().float().double()[:, None], ang.sin().float().double()[:, None]

    def rope(z):
        a, b = z[..., :D // 2], z[..., D // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    def attention(x, p):
        q = rope((x @ w[p + "q_proj.weight"].T).view(T, H, D))
        k = rope((x @ w[p + "k_proj.weight"].T).view(T, Hkv, D))
        v = (x @ w[p + "v_proj.weight"].T).view(T, Hkv, D)
        k, v = k.repeat_interleave(H // Hkv, 1), v.repeat_interleave(H // Hkv, 1)
        sc = torch.einsum("thd,shd->hts", q, k) * D ** -0.5
        mask = torch.arange(T)[None] <= torch.arange(T)[:, None]
        o = torch.einsum("hts,shd->thd", sc.masked_fill(~mask[None], float("-inf")).softmax(-1), v)
        return o.reshape(T, H * D) @ w[p + "o_proj.weight"].T

    def routed(x, p, experts_of):
        logits = x @ w[p + "router.weight"].T
        prob, expert = logits.softmax(-1).max(-1)
        experts_of.append(expert)
        up = w[p + "up.weight"].view(cfg.experts, 24, h)
        down = w[p + "down.weight"].view(cfg.experts, h, 24)
        rows = [torch.nn.functional.gelu(x[t] @ up[expert[t]].T, approximate="tanh") @ down[expert[t]].T * prob[t]
                for t in range(T)]
        return torch.stack(rows)

    def dense(x, p):
        g, u = x @ w[p + "gate_proj.weight"].T, x @ w[p + "up_proj.weight"].T
        return (g / (1 + torch.exp(-g)) * u) @ w[p + "down_proj.weight"].T

    chosen = []
    for layer in (0, 1):
        p = f"model.layers.{layer}."
        r = r + attention(norm(r, w[p + "input_layernorm.weight"]), p + "self_attn.")
        x = norm(r, w[p + "post_attention_layernorm.weight"])
        r = r + (routed(x, p + "moe.", chosen) if layer == 0 else dense(x, p + "mlp."))
    return norm(r, w["model.norm.weight"]) @ w["lm_head.weight"].T, chosen[0]


def test_toy_routed_feed_forward_and_position_encoding_run_through_the_engine(tmp_path):
    """float32, so that the engine and the plain form route every token to the same expert."""
    import os
    from safetensors.torch import load_file
    from tinyserve_b200.config import ARCHITECTURES, EngineConfig
    from tinyserve_b200.engine.batch import StepEntry
    from tinyserve_b200.engine.runner import ModelRunner
    from tinyserve_b200.parts.base import FEED_FORWARDS, POSITION_ENCODINGS
    from tinyserve_b200.weights import write_random_model
    RoutedConfig = _register_routed()
    try:
        cfg = RoutedConfig(vocab_size=83, hidden_size=48, experts=5)
        folder = write_random_model(cfg, str(tmp_path), seed=5, store_dtype="float32")
        weights = load_file(os.path.join(folder, "model.safetensors"))
        # a router that matters: spread its logits, so that several experts are chosen
        assert weights["model.layers.0.moe.up.weight"].shape == (5 * 24, 48)
        runner = ModelRunner(EngineConfig(model=folder, dtype="float32", max_model_len=96, block_size=8,
                                          max_num_seqs=2, max_num_batched_tokens=64, num_blocks=20))
        ids = random_ids(83, 45, seed=4)
        ref, experts = _plain_routed(weights, cfg, ids)
        assert len(experts.unique()) >= 2, "the routing is not trivial"
        mgr = runner.manager
        mgr.begin("a")
        got = [runner.step([StepEntry("a", ids[:30], list(range(30)))]),
               runner.step([StepEntry("a", ids[30:32], [0, 1])])]
        got += [runner.step([StepEntry("a", [ids[t]], [0])]) for t in range(32, 45)]
        mgr.free("a")
        got = torch.cat(got).double().cpu()
        assert (got - ref).abs().max().item() < 2e-5 * ref.abs().max().item()
        mgr.check_invariants()
    finally:
        ARCHITECTURES.pop("ToyRoutedForCausalLM", None)
        FEED_FORWARDS.pop("toy_routed", None)
        POSITION_ENCODINGS.pop("toy_linear_rotary", None)


# ----------------------------------------------------------------------------- a layer on another's cache
def _register_shared():
    from tinyserve_b200.config import (LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec,
                                       register_architecture)

    @dataclass(frozen=True)
    class SharedConfig(ModelConfig):
        """Two attention layers; the second keeps no keys of its own: its queries read the first
        layer's cache (the run order says so: same cache entry, writes_cache=False)."""
        architecture: ClassVar[str] = "ToySharedCacheForCausalLM"
        vocab_size: int = 0
        hidden_size: int = 0

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["vocab_size"], raw["hidden_size"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size}

        def model_spec(self):
            h = self.hidden_size
            norm = PartSpec("rmsnorm", {"eps": 1e-6})
            attn = PartSpec("attention", {
                "hidden_size": h, "num_heads": 4, "num_kv_heads": 2, "head_dim": 32, "qk_norm": norm,
                "position": PartSpec("rotary", {"rotary_dim": 32, "theta": 1e4, "pairing": "half"})})
            ffn = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": 64, "activation": "silu"})
            layers = (LayerSpec(attn, ffn, norm), LayerSpec(attn, ffn, norm))
            order = (LayerCall(0, 0), LayerCall(1, 0, writes_cache=False))
            return ModelSpec(self.vocab_size, h, layers, order, norm, True)

    register_architecture(SharedConfig.architecture, SharedConfig)
    return SharedConfig


def _plain_shared(weights, cfg, ids):
    w = {k: v.double() for k, v in weights.items()}
    T, H, Hkv, D = len(ids), 4, 2, 32
    norm = lambda x, wt: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * wt
    r = w["model.embed_tokens.weight"][torch.tensor(ids)]
    inv = 1.0 / 1e4 ** (torch.arange(0, D, 2, dtype=torch.float64) / D)
    ang = torch.outer(torch.arange(T, dtype=torch.float64), inv)
    c, s = ang.cos().float().double()[:, None], ang.sin().float().double()[:, None]

    def rope(z):
        a, b = z[..., :D // 2], z[..., D // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    kept = {}
    for layer in (0, 1):
        p = f"model.layers.{layer}."
        x = norm(r, w[p + "input_layernorm.weight"])
        q = rope(norm((x @ w[p + "self_attn.q_proj.weight"].T).view(T, H, D), w[p + "self_attn.q_norm.weight"]))
        if layer == 0:
            kept["k"] = rope(norm((x @ w[p + "self_attn.k_proj.weight"].T).view(T, Hkv, D), w[p + "self_attn.k_norm.weight"]))
            kept["v"] = (x @ w[p + "self_attn.v_proj.weight"].T).view(T, Hkv, D)
        k, v = kept["k"].repeat_interleave(H // Hkv, 1), kept["v"].repeat_interleave(H // Hkv, 1)
        sc = torch.einsum("thd,shd->hts", q, k) * D ** -0.5
        mask = torch.arange(T)[None] <= torch.arange(T)[:, None]
        o = torch.einsum("hts,shd->thd", sc.masked_fill(~mask[None], float("-inf")).softmax(-1), v).reshape(T, H * D)
        r = r + o @ w[p + "self_attn.o_proj.weight"].T
        x = norm(r, w[p + "post_attention_layernorm.weight"])
        g, u = x @ w[p + "mlp.gate_proj.weight"].T, x @ w[p + "mlp.up_proj.weight"].T
        r = r + (g / (1 + torch.exp(-g)) * u) @ w[p + "mlp.down_proj.weight"].T
    return norm(r, w["model.norm.weight"]) @ w["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 3e-2)])
def test_a_layer_reads_another_layers_cache(dtype, tol, tmp_path):
    import os
    from safetensors.torch import load_file
    from tinyserve_b200.config import ARCHITECTURES, EngineConfig
    from tinyserve_b200.engine.batch import StepEntry
    from tinyserve_b200.engine.runner import ModelRunner
    from tinyserve_b200.weights import write_random_model
    SharedConfig = _register_shared()
    try:
        cfg = SharedConfig(vocab_size=71, hidden_size=64)
        folder = write_random_model(cfg, str(tmp_path), seed=9)
        weights = load_file(os.path.join(folder, "model.safetensors"))
        runner = ModelRunner(EngineConfig(model=folder, dtype=dtype, max_model_len=96, block_size=8,
                                          max_num_seqs=2, max_num_batched_tokens=64, num_blocks=20))
        assert len(runner.model.cache_entries) == 1, "one cache entry for both layers"
        ids = random_ids(71, 40, seed=6)
        ref = _plain_shared(weights, cfg, ids)
        mgr = runner.manager
        mgr.begin("a")
        got = [runner.step([StepEntry("a", ids[:25], list(range(25)))])]
        got += [runner.step([StepEntry("a", [ids[t]], [0])]) for t in range(25, 40)]
        mgr.free("a")
        got = torch.cat(got).double().cpu()
        assert (got - ref).abs().max().item() < tol * ref.abs().max().item()
    finally:
        ARCHITECTURES.pop("ToySharedCacheForCausalLM", None)
