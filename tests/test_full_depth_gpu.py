"""The true 32-bit path at full size: all 36 layers of the Qwen3-8B shapes, the whole vocabulary
of 151,936, 4,096 tokens of context, random weights.  The logits of the last positions are held
against the plain implementation, which runs on the device in float64, under four schedules:
the prompt whole; all but 32 tokens in one step and the rest one by one; shrinking portions; and
mixed steps with two portions beside two decoding requests.

The bar is a largest absolute logit difference of 1e-4.  The weights (16 GB in bfloat16) are drawn
on the device and written one file per layer by this test's own writer, under the checkpoint's
tensor names; engine (33 GB in float32) and plain implementation (66 GB in float64) both read
that folder.  This one test takes a few minutes."""
import json
import os
import shutil
import tempfile

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

import plain_qwen3 as plain
from helpers import lines_of, random_ids

pytestmark = pytest.mark.gpu

SHAPES = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096, num_hidden_layers=36,
              num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
              vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
BAR = 1e-4


def write_folder(folder, raw, seed):
    """N(0, 0.02) matrices, norm weights 1 + U(-0.1, 0.1), bfloat16, one file per layer."""
    h, L, V = raw["hidden_size"], raw["num_hidden_layers"], raw["vocab_size"]
    H, Hkv, D, I = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"], raw["intermediate_size"]
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(raw, fh)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    mat = lambda r, c: (torch.randn(r, c, generator=gen, device="cuda") * 0.02).to(torch.bfloat16).cpu()
    vec = lambda n: (0.9 + 0.2 * torch.rand(n, generator=gen, device="cuda")).to(torch.bfloat16).cpu()
    save_file({"model.embed_tokens.weight": mat(V, h), "model.norm.weight": vec(h), "lm_head.weight": mat(V, h)},
              os.path.join(folder, "model-ends.safetensors"))
    for i in range(L):
        p = f"model.layers.{i}."
        save_file({p + "self_attn.q_proj.weight": mat(H * D, h), p + "self_attn.k_proj.weight": mat(Hkv * D, h),
                   p + "self_attn.v_proj.weight": mat(Hkv * D, h), p + "self_attn.o_proj.weight": mat(h, H * D),
                   p + "self_attn.q_norm.weight": vec(D), p + "self_attn.k_norm.weight": vec(D),
                   p + "mlp.gate_proj.weight": mat(I, h), p + "mlp.up_proj.weight": mat(I, h),
                   p + "mlp.down_proj.weight": mat(h, I), p + "input_layernorm.weight": vec(h),
                   p + "post_attention_layernorm.weight": vec(h)},
                  os.path.join(folder, f"model-layer{i:02d}.safetensors"))


def scratch_folder(need_bytes):
    best = max((d for d in (tempfile.gettempdir(), "/dev/shm") if os.path.isdir(d) and os.access(d, os.W_OK)),
               key=lambda d: shutil.disk_usage(d).free)
    if shutil.disk_usage(best).free < need_bytes:
        pytest.skip(f"no temporary folder with {need_bytes >> 30} GiB free")
    return tempfile.mkdtemp(prefix="tinyserve_full_", dir=best)


def test_32_bit_logits_at_full_depth_and_4096_context():
    from tinyserve_b200.engine import replay
    free, _ = torch.cuda.mem_get_info()
    if free < 120 << 30:
        pytest.skip("needs 120 GB of device memory (engine in float32 beside the plain model in float64)")
    V, T, tail = SHAPES["vocab_size"], 4096, 32
    folder = scratch_folder(18 << 30)
    try:
        write_folder(folder, SHAPES, seed=5)
        ids = {"a": random_ids(V, T, seed=1), "b": random_ids(V, 1000, seed=2),
               "c": random_ids(V, 203, seed=3), "d": random_ids(V, 263, seed=4)}
        # rows of every request whose logits are compared
        rows = {"a": list(range(T - 64, T)), "b": list(range(980, 1000)), "c": [200, 201, 202], "d": [260, 261, 262]}
        cfg, weights = plain.load_folder(folder, dtype=torch.float64, device="cuda")
        ref = {}
        with torch.no_grad():
            for rid, seq in ids.items():
                hidden = plain.hidden_states(cfg, weights, seq)[rows[rid]]
                ref[rid] = (hidden @ weights["lm_head.weight"].T).cpu()
        del weights, hidden
        torch.cuda.empty_cache()
        runner = replay.make_runner(folder, "float32", 4096 + 1024 + 256 + 320)
    finally:
        shutil.rmtree(folder, ignore_errors=True)

    def entry(rid, a, b):
        return {"id": rid, "tokens": ids[rid][a:b], "want": [j - a for j in rows[rid] if a <= j < b]}

    cuts = [0, 2000, 3200, 3800, 4050, 4090, 4094, T]
    schedules = {
        "whole": [{"step": 0, "entries": [entry("a", 0, T)], "end": ["a"]}],
        "last 32 one by one": [{"step": 0, "entries": [entry("a", 0, T - tail)], "end": []}] +
                              [{"step": 1 + i, "entries": [entry("a", T - tail + i, T - tail + i + 1)],
                                "end": ["a"] if i == tail - 1 else []} for i in range(tail)],
        "shrinking portions": [{"step": i, "entries": [entry("a", a, b)], "end": ["a"] if b == T else []}
                               for i, (a, b) in enumerate(zip(cuts, cuts[1:]))],
        "mixed": [
            {"step": 0, "entries": [entry("c", 0, 200), entry("d", 0, 260), entry("b", 0, 600)], "end": []},
            {"step": 1, "entries": [entry("a", 0, 1500), entry("c", 200, 201), entry("b", 600, 900),
                                    entry("d", 260, 261)], "end": []},
            {"step": 2, "entries": [entry("c", 201, 202), entry("a", 1500, 4032), entry("d", 261, 262),
                                    entry("b", 900, 1000)], "end": ["b"]},
            {"step": 3, "entries": [entry("d", 262, 263), entry("a", 4032, T), entry("c", 202, 203)],
             "end": ["a", "c", "d"]},
        ],
    }
    assert sum(len(e["tokens"]) > 1 for e in schedules["mixed"][1]["entries"]) == 2
    assert sum(len(e["tokens"]) == 1 for e in schedules["mixed"][1]["entries"]) == 2
    report = {}
    for name, steps in schedules.items():
        out = tempfile.mkdtemp()
        try:
            replay.replay(runner, lines_of(steps), out, lambda msg: None)
            got = {}
            for s in steps:
                n = sum(len(e["want"]) for e in s["entries"])
                if not n:
                    continue
                data = torch.from_numpy(np.fromfile(os.path.join(out, f"{s['step']}.f32"), dtype="<f4").reshape(n, V))
                k = 0
                for e in s["entries"]:
                    if e["want"]:
                        got.setdefault(e["id"], []).append(data[k:k + len(e["want"])])
                        k += len(e["want"])
        finally:
            shutil.rmtree(out, ignore_errors=True)
        worst = 0.0
        for rid, parts in got.items():
            mine = torch.cat(parts).double()
            assert mine.shape == ref[rid].shape
            worst = max(worst, (mine - ref[rid]).abs().max().item())
        assert set(got) == ({"a"} if name != "mixed" else set(ids))
        report[name] = worst
        assert not runner.manager.requests
    scale = max(r.abs().max().item() for r in ref.values())
    print(f"[measured] 36 layers, float32, largest |logit difference| per schedule: "
          + ", ".join(f"{k} {v:.2e}" for k, v in report.items()) + f" (largest |logit| {scale:.2f})")
    for name, worst in report.items():
        assert worst <= BAR, f"{name}: largest logit difference {worst:.3e} exceeds {BAR}"
