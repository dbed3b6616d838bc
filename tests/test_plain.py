"""The plain implementation itself (no GPU): against tinyserve's own model code through the
stored outputs of tests/golden/make_reference_golden.py, and its parts against each other."""
import os

import numpy as np
import pytest
import torch
from safetensors.torch import load_file

import plain_qwen3 as plain
from helpers import make_model_dir, random_ids, tiny_config_dict

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_the_reference_model(name):
    """tinyserve's own serve.Model ran once on these very tensors (they are stored with its
    logits: tests/golden/make_reference_golden.py); the plain implementation must agree."""
    gold = np.load(os.path.join(GOLDEN, f"reference_logits_{name}.npz"))
    weights = {key[2:]: torch.from_numpy(gold[key]).view(torch.bfloat16).double()
               for key in gold.files if key.startswith("w:")}
    assert len(weights) > 10 and "model.embed_tokens.weight" in weights
    cfg = plain.normalise_config(tiny_config_dict(name))
    ours = plain.logits(cfg, weights, gold["ids"].tolist())
    ref = torch.from_numpy(gold["logits"]).double()
    assert ref.abs().max() > 0.1
    assert (ours - ref).abs().max().item() < 2e-6      # the reference ran in float32


def test_window_equals_full_attention_when_it_covers_everything():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(20, 6, 8, generator=g, dtype=torch.float64),
               torch.randn(20, 2, 8, generator=g, dtype=torch.float64),
               torch.randn(20, 2, 8, generator=g, dtype=torch.float64))
    full = plain.causal_attention(q, k, v, 0.3)
    assert torch.allclose(full, plain.causal_attention(q, k, v, 0.3, window=20))
    w5 = plain.causal_attention(q, k, v, 0.3, window=5)
    assert torch.allclose(w5[:5], full[:5]) and not torch.allclose(w5[5:], full[5:])
    # the query at position 9 with window 5 sees keys 5..9 only
    alone = plain.causal_attention(q[5:10], k[5:10], v[5:10], 0.3)
    assert torch.allclose(w5[9], alone[4])


def test_prefix_invariance_and_greedy(tmp_path):
    folder = make_model_dir(tmp_path, "C", seed=4)
    cfg, weights = plain.load_folder(folder)
    ids = random_ids(cfg["vocab_size"], 60, seed=1)
    whole = plain.logits(cfg, weights, ids)
    assert torch.allclose(whole[:33], plain.logits(cfg, weights, ids[:33]), atol=1e-12)
    out = plain.greedy_generate(cfg, weights, ids[:5], 3)
    assert len(out) == 3 and out[0] == int(whole[4].argmax())
    # the second token continues from the first one it chose, not from the prompt's own next token
    assert out[1] == int(plain.logits(cfg, weights, ids[:5] + out[:1])[-1].argmax())


def test_rope_and_norm_formulas():
    cos, sin = plain.rope_tables(8, 10000.0, 4, torch.float64)
    assert cos.shape == (4, 4) and torch.allclose(cos[0], torch.ones(4, dtype=torch.float64))
    x = torch.arange(16, dtype=torch.float64).view(1, 2, 8)
    y = plain.apply_rope(x, cos[3:4], sin[3:4])
    assert torch.allclose(y[0, 0, 0], x[0, 0, 0] * cos[3, 0] - x[0, 0, 4] * sin[3, 0])
    assert torch.allclose(y[0, 0, 4], x[0, 0, 4] * cos[3, 0] + x[0, 0, 0] * sin[3, 0])
    n = plain.rms_norm(torch.tensor([[3.0, 4.0]]), torch.tensor([2.0, 0.5]), 0.0)
    assert torch.allclose(n, torch.tensor([[3.0 / 12.5 ** 0.5 * 2.0, 4.0 / 12.5 ** 0.5 * 0.5]]))


def test_sampling_pieces():
    row = torch.tensor([2.0, -1.0, 0.5, 0.0])
    assert torch.allclose(plain.repetition_penalty(row, [0, 1, 1], 1.1),
                          torch.tensor([2.0 / 1.1, -1.1, 0.5, 0.0]))
    kept = plain.top_k_top_p_mask(torch.tensor([1.0, 3.0, 2.0, 0.0]), 1.0, 3, 1.0)
    assert torch.isinf(kept[3]) and not torch.isinf(kept[:3]).any()
    kept = plain.top_k_top_p_mask(torch.tensor([1.0, 3.0, 2.0, 0.0]), 1.0, -1, 0.7)
    assert [bool(torch.isinf(v)) for v in kept] == [True, False, False, True]
    # Philox-4x32-10, known answer for an all-zero counter and key
    assert plain.philox4x32((0, 0, 0, 0), (0, 0)) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    g = plain.gumbel_noise(7, 3, 2, 10)
    assert g.shape == (10,) and np.isfinite(g).all()
    assert plain.sample_row(row, 0.0, 0, 0, 0) == 0
