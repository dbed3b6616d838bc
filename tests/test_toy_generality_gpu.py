"""What another architecture would need of the framework, shown with toy parts that are defined
here and registered without a change to the package:

  * a checkpoint whose tensors have other names than Qwen's: names are data of the specification;
  * a mixer that caches ONE latent vector per token (not keys and values) in pages of its own
    geometry, beside a position encoding that is learned and added to the embeddings;
  * a mixer with state of its own under an engine with CUDA graphs switched on: a part that reads
    host-side lists is not capturable, and the engine then runs it eagerly instead of replaying
    a graph with the capture's lists;
  * a norm written against the plain interface (tensors in, tensors out)."""
import os
from dataclasses import dataclass
from typing import ClassVar

import pytest
import torch
from safetensors.torch import load_file

import plain_qwen3 as plain
from helpers import random_ids

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------------------- other tensor names
def _register_renamed():
    from tinyserve_b200.config import LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec, register_architecture

    @dataclass(frozen=True)
    class RenamedConfig(ModelConfig):
        """The Qwen3 layer under a checkpoint that calls everything differently."""
        architecture: ClassVar[str] = "ToyRenamedForCausalLM"
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
                "position": PartSpec("rotary", {"rotary_dim": 32, "theta": 1e4, "pairing": "half"}),
                "names": {"q": "wq", "k": "wk", "v": "wv", "o": "wo", "q_norm": "qn", "k_norm": "kn"}})
            ffn = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": 80, "activation": "silu",
                                         "names": {"gate": "w1", "up": "w3", "down": "w2"}})
            names = {"mixer": "attn", "ffn": "ff", "input_norm": "ln1", "post_mixer_norm": "ln2"}
            layers = tuple(LayerSpec(attn, ffn, norm, names=names) for _ in range(2))
            return ModelSpec(self.vocab_size, h, layers, (LayerCall(0, 0), LayerCall(1, 1)), norm, False,
                             weight_prefix="", names={"embed": "tok_emb", "layers": "blocks.{i}",
                                                      "final_norm": "ln_f", "lm_head": "head"})

    register_architecture(RenamedConfig.architecture, RenamedConfig)
    return RenamedConfig


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 3e-2)])
def test_a_checkpoint_with_other_tensor_names(dtype, tol, tmp_path):
    from tinyserve_b200.config import ARCHITECTURES, EngineConfig
    from tinyserve_b200.engine.batch import StepEntry
    from tinyserve_b200.engine.runner import ModelRunner
    from tinyserve_b200.weights import write_random_model
    RenamedConfig = _register_renamed()
    try:
        cfg = RenamedConfig(vocab_size=91, hidden_size=64)
        folder = write_random_model(cfg, str(tmp_path), seed=2)
        weights = load_file(os.path.join(folder, "model.safetensors"))
        assert {"tok_emb.weight", "head.weight", "ln_f.weight", "blocks.1.attn.wq.weight", "blocks.0.attn.qn.weight",
                "blocks.0.ff.w3.weight", "blocks.1.ln2.weight"} <= set(weights)
        assert not any(k.startswith("model.") for k in weights)
        # the same model under Qwen's names, for the plain implementation
        rename = {"tok_emb": "model.embed_tokens", "head": "lm_head", "ln_f": "model.norm", "blocks.": "model.layers.",
                  ".attn.": ".self_attn.", ".ff.": ".mlp.", ".wq.": ".q_proj.", ".wk.": ".k_proj.", ".wv.": ".v_proj.",
                  ".wo.": ".o_proj.", ".qn.": ".q_norm.", ".kn.": ".k_norm.", ".w1.": ".gate_proj.",
                  ".w3.": ".up_proj.", ".w2.": ".down_proj.", ".ln1.": ".input_layernorm.",
                  ".ln2.": ".post_attention_layernorm."}
        qwen = {}
        for key, value in weights.items():
            for a, b in rename.items():
                key = key.replace(a, b)
            qwen[key] = value.double()
        pcfg = plain.normalise_config(dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                                           num_key_value_heads=2, head_dim=32, intermediate_size=80, vocab_size=91,
                                           rms_norm_eps=1e-6, rope_theta=1e4, tie_word_embeddings=False))
        ids = random_ids(91, 37, seed=3)
        ref = plain.logits(pcfg, qwen, ids)
        runner = ModelRunner(EngineConfig(model=folder, dtype=dtype, max_model_len=64, block_size=8,
                                          max_num_seqs=2, max_num_batched_tokens=64, num_blocks=12))
        runner.manager.begin("a")
        got = [runner.step([StepEntry("a", ids[:30], list(range(30)))])]
        got += [runner.step([StepEntry("a", [ids[t]], [0])]) for t in range(30, 37)]
        got = torch.cat(got).double().cpu()
        assert (got - ref).abs().max().item() < tol * ref.abs().max().item()
    finally:
        ARCHITECTURES.pop("ToyRenamedForCausalLM", None)


# ----------------------------------------------------------------------------- one latent per token
def _register_latent():
    from tinyserve_b200.config import LayerCall, LayerSpec, ModelConfig, ModelSpec, PartSpec, register_architecture
    from tinyserve_b200.parts import CacheSpec, CacheTensor, Mixer, Norm, ParamSpec
    from tinyserve_b200.parts.base import (PositionEncoding, register_mixer, register_norm,
                                           register_position_encoding)

    class LatentMixer(Mixer):
        """Caches one latent c_t = x_t Wc^T of ``rank`` numbers per token.  The query q_t = x_t Wq^T
        attends to the latents of its request up to its own position; out_t = (sum_j p_tj c_j) Wo^T."""
        tree_name = "latent"

        def __init__(self, hidden_size, rank):
            super().__init__()
            self.h, self.r = hidden_size, rank

        def param_specs(self):
            return {"wc.weight": ParamSpec((self.r, self.h)), "wq.weight": ParamSpec((self.r, self.h)),
                    "wo.weight": ParamSpec((self.h, self.r))}

        def cache_spec(self):
            return CacheSpec("full", tensors=(CacheTensor("latent", 1, self.r),))

        def forward(self, h, ctx, call):
            cache = ctx.cache(call.cache)
            view = ctx.group(cache.group)
            pool = cache.tensors["latent"]                  # [page, 1, slot, rank]
            x = h.float()
            c = x @ self.w["wc.weight"].float().T
            q = x @ self.w["wq.weight"].float().T
            slots = view.slot_mapping.long()
            flat = pool.view(-1, self.r)                    # row page * page_size + slot (one head)
            keep = slots >= 0
            flat[slots[keep]] = c[keep].to(pool.dtype)       # page * page_size + slot, one head
            out = torch.zeros_like(x[:, :self.r])
            cu, kv = ctx.host["cu_q"], ctx.host["kv_lens"]
            for b in range(ctx.num_requests):
                n = cu[b + 1] - cu[b]
                if n == 0:
                    continue
                pages = view.block_table[b].long()
                j = torch.arange(kv[b], device=h.device)
                lat = flat[pages[j // view.page_size] * view.page_size + j % view.page_size].float()
                sc = q[cu[b]:cu[b + 1]] @ lat.T * self.r ** -0.5
                pos = torch.arange(kv[b] - n, kv[b], device=h.device)
                sc = sc.masked_fill(j[None] > pos[:, None], float("-inf"))
                out[cu[b]:cu[b + 1]] = sc.softmax(-1) @ lat
            return (out @ self.w["wo.weight"].float().T).to(h.dtype)

    class LearnedPositions(PositionEncoding):
        """A table of one vector per absolute position, added to the embeddings."""
        capturable = True

        def __init__(self, hidden_size, positions):
            super().__init__()
            self.h, self.n = hidden_size, positions

        def param_specs(self):
            return {"weight": ParamSpec((self.n, self.h))}

        def add_to_embeddings(self, residual, ctx):
            residual += self.w["weight"][ctx.positions.long()].float()

    class MeanNorm(Norm):
        """LayerNorm without bias, written against the plain interface: y = (x - mean) / std * w."""

        def __init__(self, dim, eps):
            super().__init__()
            self.dim, self.eps = dim, eps

        def param_specs(self):
            return {"weight": ParamSpec((self.dim,), role="vector", init="norm_weight")}

        def prepare(self, runtime):
            self.dtype = runtime.dtype

        def forward(self, x, out=None):
            xf = x.float()
            xf = xf - xf.mean(-1, keepdim=True)
            return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.w["weight"].float()).to(x.dtype)

        def add_forward(self, x, residual, rows=None):
            assert x is None or isinstance(x, torch.Tensor), "a norm sees plain tensors"
            if rows is not None:
                picked = residual[rows.long()] + (x[rows.long()].float() if x is not None else 0)
                return self.forward(picked).to(self.dtype)
            if x is not None:
                residual += x.float()
            return self.forward(residual).to(self.dtype)

    @dataclass(frozen=True)
    class LatentConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyLatentForCausalLM"
        vocab_size: int = 0
        hidden_size: int = 0
        rank: int = 0
        positions: int = 0

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["vocab_size"], raw["hidden_size"], raw["rank"], raw["positions"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size,
                    "hidden_size": self.hidden_size, "rank": self.rank, "positions": self.positions}

        def model_spec(self):
            h = self.hidden_size
            norm = PartSpec("toy_mean_norm", {"eps": 1e-5})
            rms = PartSpec("rmsnorm", {"eps": 1e-5})
            ffn = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": 2 * h, "activation": "silu"})
            latent = LayerSpec(PartSpec("toy_latent", {"hidden_size": h, "rank": self.rank}), ffn, norm)
            attn = LayerSpec(PartSpec("attention", {"hidden_size": h, "num_heads": 2, "num_kv_heads": 1,
                                                    "head_dim": 16}), ffn, rms)
            return ModelSpec(self.vocab_size, h, (latent, attn, latent), (LayerCall(0, 0), LayerCall(1, 1), LayerCall(2, 2)),
                             rms, True, embedding_position=PartSpec("toy_learned_positions",
                                                                    {"hidden_size": h, "positions": self.positions}))

    register_mixer("toy_latent", LatentMixer)
    register_norm("toy_mean_norm", MeanNorm)
    register_position_encoding("toy_learned_positions", LearnedPositions)
    register_architecture(LatentConfig.architecture, LatentConfig)
    return LatentConfig


def _plain_latent(weights, cfg, ids):
    w = {k: v.double() for k, v in weights.items()}
    T, h, r = len(ids), cfg.hidden_size, cfg.rank
    rms = lambda x, wt: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * wt

    def mean_norm(x, wt):
        x = x - x.mean(-1, keepdim=True)
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * wt

    mask = torch.arange(T)[None] > torch.arange(T)[:, None]
    x = w["model.embed_tokens.weight"][torch.tensor(ids)] + w["model.embed_positions.weight"][:T]
    for layer, kind in ((0, "latent"), (1, "attn"), (2, "latent")):
        p = f"model.layers.{layer}."
        norm = mean_norm if kind == "latent" else rms
        y = norm(x, w[p + "input_layernorm.weight"])
        if kind == "latent":
            c, q = y @ w[p + "latent.wc.weight"].T, y @ w[p + "latent.wq.weight"].T
            sc = (q @ c.T * r ** -0.5).masked_fill(mask, float("-inf"))
            x = x + (sc.softmax(-1) @ c) @ w[p + "latent.wo.weight"].T
        else:
            q = (y @ w[p + "self_attn.q_proj.weight"].T).view(T, 2, 16)
            k = (y @ w[p + "self_attn.k_proj.weight"].T).view(T, 1, 16)
            v = (y @ w[p + "self_attn.v_proj.weight"].T).view(T, 1, 16)
            sc = torch.einsum("thd,sd->hts", q, k[:, 0]) * 16 ** -0.5
            o = torch.einsum("hts,sd->thd", sc.masked_fill(mask[None], float("-inf")).softmax(-1), v[:, 0])
            x = x + o.reshape(T, 32) @ w[p + "self_attn.o_proj.weight"].T
        y = norm(x, w[p + "post_attention_layernorm.weight"])
        g, u = y @ w[p + "mlp.gate_proj.weight"].T, y @ w[p + "mlp.up_proj.weight"].T
        x = x + (g / (1 + torch.exp(-g)) * u) @ w[p + "mlp.down_proj.weight"].T
    return rms(x, w["model.norm.weight"]) @ w["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 3e-2)])
def test_a_latent_cache_learned_positions_and_a_plain_norm(dtype, tol, tmp_path):
    from tinyserve_b200.config import ARCHITECTURES, EngineConfig
    from tinyserve_b200.engine.batch import StepEntry
    from tinyserve_b200.engine.runner import ModelRunner
    from tinyserve_b200.parts.base import MIXERS, NORMS, POSITION_ENCODINGS
    from tinyserve_b200.weights import write_random_model
    LatentConfig = _register_latent()
    try:
        cfg = LatentConfig(vocab_size=77, hidden_size=48, rank=24, positions=96)
        folder = write_random_model(cfg, str(tmp_path), seed=8)
        weights = load_file(os.path.join(folder, "model.safetensors"))
        assert weights["model.embed_positions.weight"].shape == (96, 48)
        runner = ModelRunner(EngineConfig(model=folder, dtype=dtype, max_model_len=96, block_size=8,
                                          max_num_seqs=3, max_num_batched_tokens=64, num_blocks=16))
        model = runner.model
        # two page pools: latents (one head of 24 numbers per token, two layers) and keys/values
        assert [[(t.name, t.heads, t.width) for t in g.tensors] for g in model.cache_groups] == \
            [[("latent", 1, 24)], [("k", 1, 16), ("v", 1, 16)]]
        assert model.group_sizes == [2, 1] and not model.capturable
        assert runner.device_cache.pools[0]["latent"].shape == (2, 17, 1, 8, 24)
        element = 4 if dtype == "float32" else 2
        assert runner.device_cache.bytes_per_page(model, 8, element) == [2 * 24 * 8 * element, 2 * 16 * 8 * element]
        a, b = random_ids(77, 60, seed=1), random_ids(77, 21, seed=2)
        ref_a, ref_b = _plain_latent(weights, cfg, a), _plain_latent(weights, cfg, b)
        mgr = runner.manager
        mgr.begin("a"); mgr.begin("b")
        got_a = [runner.step([StepEntry("a", a[:33], list(range(33)))])]
        out = runner.step([StepEntry("b", b[:19], list(range(19))), StepEntry("a", a[33:35], [0, 1])])
        got_b, _ = [out[:19]], got_a.append(out[19:])
        for t in range(2):
            out = runner.step([StepEntry("a", a[35 + 12 * t:47 + 12 * t], list(range(12))), StepEntry("b", [b[19 + t]], [0])])
            got_a.append(out[:12]); got_b.append(out[12:])
        got_a.append(runner.step([StepEntry("a", [a[59]], [0])]))
        mgr.free("a"); mgr.free("b")
        for got, ref in ((torch.cat(got_a), ref_a), (torch.cat(got_b), ref_b)):
            assert (got.double().cpu() - ref).abs().max().item() < tol * ref.abs().max().item()
        mgr.check_invariants()
    finally:
        ARCHITECTURES.pop("ToyLatentForCausalLM", None)
        MIXERS.pop("toy_latent", None)
        NORMS.pop("toy_mean_norm", None)
        POSITION_ENCODINGS.pop("toy_learned_positions", None)


# ----------------------------------------------------------------------------- state under graphs
def test_a_mixer_that_reads_host_lists_is_never_replayed_from_a_graph(tmp_path):
    """The toy mixer with state (test_toy_parts_gpu.py) reads the step's host-side lists.  With
    CUDA graphs on, the engine must not capture it: generation gives the tokens of the run
    without graphs, and of the plain form."""
    import test_toy_parts_gpu as toy
    from tinyserve_b200 import LLM, SamplingParams
    from tinyserve_b200.config import ARCHITECTURES
    from tinyserve_b200.parts.base import MIXERS
    from tinyserve_b200.weights import write_random_model
    ToyConfig = toy._register()
    try:
        cfg = ToyConfig(vocab_size=97, hidden_size=40, decay=0.7, heads=3)
        folder = write_random_model(cfg, str(tmp_path), seed=3, store_dtype="float32")
        weights = load_file(os.path.join(folder, "model.safetensors"))
        prompts = [random_ids(97, 9, seed=1), random_ids(97, 30, seed=2), random_ids(97, 2, seed=3)]
        params = SamplingParams(temperature=0.0, max_tokens=12, repetition_penalty=1.0, ignore_eos=True)
        outs = {}
        for graphs in (True, False):
            llm = LLM(folder, dtype="float32", max_model_len=64, block_size=8, max_num_seqs=2,
                      max_num_batched_tokens=16, num_blocks=20, use_cuda_graphs=graphs)
            assert not llm.runner.model.capturable and not llm.runner.graphs
            outs[graphs] = [o.token_ids for o in llm.generate(prompts, params)]
        assert outs[True] == outs[False]
        for prompt, tokens in zip(prompts, outs[True]):
            ids = list(prompt)
            for tok in tokens:
                assert tok == int(toy._plain_toy(weights, cfg, ids)[-1].argmax())
                ids.append(tok)
    finally:
        ARCHITECTURES.pop("ToyDecayForCausalLM", None)
        MIXERS.pop("toy_decay", None)
