"""A plain, slow Qwen3 dense decoder: whole sequences, no cache, one function per part.

It shares no code with ``tinyserve_b200``: it reads ``config.json`` and
``model.safetensors`` of a model folder by itself and evaluates the formulas of
priyammaz/tinyserve's ``serve.py`` (cited at each function by file:line) with
torch tensor arithmetic on the CPU.  ``tests/golden/make_reference_golden.py``
compared it once with tinyserve's own ``serve.Model`` on the CPU; the outputs of
that run are under ``tests/golden/``.

All arithmetic runs in ``dtype`` (float64 by default, so that the engine's own
32-bit rounding is the only error that a comparison shows); the rotary tables are
rounded to float32 first, as serve.py:1227-1228 does.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np
import torch
from safetensors import safe_open


# ----------------------------------------------------------------------------- parts

def rms_norm(x, weight, eps):
    """serve.py:806-809: x * rsqrt(mean(x^2, -1) + eps) * weight."""
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight


def rope_tables(rotary_dim, theta, num_positions, dtype):
    """serve.py:1225-1228: inv_freq = 1/theta^(2i/D) in float64, cos/sin stored as float32."""
    inv_freq = 1.0 / theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float64) / rotary_dim)
    freqs = torch.outer(torch.arange(num_positions, dtype=torch.float64), inv_freq)
    return freqs.cos().float().to(dtype), freqs.sin().float().to(dtype)


def apply_rope(x, cos, sin):
    """serve.py:811-814, rotate-half: pairs (i, i + D/2); x is [T, heads, D], cos/sin [T, D/2]."""
    x1, x2 = x.chunk(2, dim=-1)
    cos, sin = cos[:, None], sin[:, None]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)


def causal_attention(q, k, v, scale, window=0):
    """serve.py:639-688 for one request that is present whole (q_len == kv_len).

    q [T, H, D], k and v [T, Hkv, D].  Query head g uses KV head g // (H // Hkv)
    (serve.py:673-674); key j is visible to the query at position p iff j <= p
    (serve.py:676-677).  ``window`` > 0 further hides keys with j <= p - window
    (tinyserve has no window; see Qwen3Config).  Softmax over the visible keys.
    """
    T, H, D = q.shape
    group = H // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("thd,shd->hts", q, k) * scale
    pos = torch.arange(T, device=q.device)
    visible = pos[None, :] <= pos[:, None]
    if window > 0:
        visible &= pos[None, :] > pos[:, None] - window
    scores = scores.masked_fill(~visible[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hts,shd->thd", probs, v)


def attention_block(h, w, prefix, cfg, cos, sin, window):
    """serve.py:843-883: q/k/v projections, per-head q_norm/k_norm before RoPE
    (serve.py:873-876), attention with scale head_dim**-0.5 (serve.py:906), o_proj."""
    T = h.shape[0]
    H, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    q = h @ w[prefix + "q_proj.weight"].T
    k = h @ w[prefix + "k_proj.weight"].T
    v = h @ w[prefix + "v_proj.weight"].T
    if prefix + "q_proj.bias" in w:
        q = q + w[prefix + "q_proj.bias"]
        k = k + w[prefix + "k_proj.bias"]
        v = v + w[prefix + "v_proj.bias"]
    q, k, v = q.view(T, H, D), k.view(T, Hkv, D), v.view(T, Hkv, D)
    q = rms_norm(q, w[prefix + "q_norm.weight"], cfg["rms_norm_eps"])
    k = rms_norm(k, w[prefix + "k_norm.weight"], cfg["rms_norm_eps"])
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    out = causal_attention(q, k, v, D ** -0.5, window)
    return out.reshape(T, H * D) @ w[prefix + "o_proj.weight"].T


def swiglu_mlp(h, w, prefix):
    """serve.py:915-919: down(silu(gate(h)) * up(h))."""
    gate = h @ w[prefix + "gate_proj.weight"].T
    up = h @ w[prefix + "up_proj.weight"].T
    return (torch.nn.functional.silu(gate) * up) @ w[prefix + "down_proj.weight"].T


def decoder_layer(r, w, i, cfg, cos, sin, window):
    """serve.py:1177-1193 written out: r1 = r0 + attn(norm1(r0)); r2 = r1 + mlp(norm2(r1))."""
    p = f"model.layers.{i}."
    h = rms_norm(r, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    r = r + attention_block(h, w, p + "self_attn.", cfg, cos, sin, window)
    h = rms_norm(r, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    return r + swiglu_mlp(h, w, p + "mlp.")


# ----------------------------------------------------------------------------- model

def normalise_config(raw):
    """The keys serve.py reads for qwen3, with its defaults (serve.py:819-824, 1209-1223)."""
    cfg = dict(raw)
    cfg.setdefault("num_key_value_heads", cfg["num_attention_heads"])
    if not cfg.get("head_dim"):
        cfg["head_dim"] = cfg["hidden_size"] // cfg["num_attention_heads"]
    rope = cfg.get("rope_parameters") or cfg.get("rope_scaling") or {}
    cfg["rope_theta"] = cfg.get("rope_theta") or rope.get("rope_theta", 10000.0)
    cfg.setdefault("tie_word_embeddings", False)
    return cfg


def layer_window(cfg, i):
    if not cfg.get("use_sliding_window"):
        return 0
    types = cfg.get("layer_types")
    if types:
        return cfg["sliding_window"] if types[i] == "sliding_attention" else 0
    mwl = cfg.get("max_window_layers")
    if mwl is None:
        mwl = cfg["num_hidden_layers"]
    return cfg["sliding_window"] if i >= mwl else 0


def load_folder(model_dir, dtype=torch.float64, device="cpu"):
    """config.json and every tensor of the folder's safetensors files, as ``dtype`` on ``device``
    (each tensor moves before it is converted, so that a large model is widened on the device)."""
    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = normalise_config(json.load(fh))
    weights = {}
    for name in sorted(os.listdir(model_dir)):
        if name.endswith(".safetensors"):
            with safe_open(os.path.join(model_dir, name), "pt", device="cpu") as fh:
                for key in fh.keys():
                    weights[key] = fh.get_tensor(key).to(device).to(dtype)
    return cfg, weights


def hidden_states(cfg, w, token_ids, dtype=torch.float64):
    """serve.py:1253-1258: embed, the layers, last residual add + final norm. Returns [T, h]."""
    device = w["model.embed_tokens.weight"].device       # CPU in most tests; a GPU for large shapes
    ids = torch.as_tensor(token_ids, dtype=torch.long).to(device)
    T = ids.shape[0]
    cos, sin = (t.to(device) for t in rope_tables(cfg["head_dim"], cfg["rope_theta"], T, dtype))
    r = w["model.embed_tokens.weight"][ids]                       # serve.py:1239
    for i in range(cfg["num_hidden_layers"]):
        r = decoder_layer(r, w, i, cfg, cos, sin, layer_window(cfg, i))
    return rms_norm(r, w["model.norm.weight"], cfg["rms_norm_eps"])


def logits(cfg, w, token_ids, dtype=torch.float64):
    """serve.py:1260-1263: hidden @ W.T with W = embed_tokens (tied) or lm_head. [T, V]."""
    hidden = hidden_states(cfg, w, token_ids, dtype)
    head = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return hidden @ head.T


def greedy_generate(cfg, w, prompt, num_tokens, dtype=torch.float64):
    """serve.py:1521-1522 (argmax) in a loop that recomputes the whole sequence each token."""
    ids = list(prompt)
    for _ in range(num_tokens):
        ids.append(int(logits(cfg, w, ids, dtype)[-1].argmax()))
    return ids[len(prompt):]


# ----------------------------------------------------------------------------- sampling

def repetition_penalty(row, recent_ids, penalty):
    """serve.py:1488-1497: every distinct recent token: logit > 0 ? logit / p : logit * p."""
    row = row.clone()
    for t in set(recent_ids):
        row[t] = row[t] / penalty if row[t] > 0 else row[t] * penalty
    return row


def top_k_top_p_mask(row, temperature, top_k, top_p):
    """serve.py:1575-1582: sort descending, /temperature, hide ranks >= k, softmax, hide
    tokens whose preceding mass exceeds top_p.  Returns the kept logits (others -inf)."""
    V = row.shape[0]
    sorted_logits, idx = torch.sort(row.double(), descending=True, stable=True)
    sorted_logits = sorted_logits / temperature
    if 0 < top_k < V:
        sorted_logits[top_k:] = float("-inf")
    probs = torch.softmax(sorted_logits, -1)
    drop = probs.cumsum(-1) - probs > top_p
    sorted_logits[drop] = float("-inf")
    out = torch.full_like(sorted_logits, float("-inf"))
    out[idx] = sorted_logits
    return out


def _mulhilo(a, b):
    p = int(a) * int(b)
    return (p >> 32) & 0xFFFFFFFF, p & 0xFFFFFFFF


def philox4x32(counter, key):
    """Philox-4x32-10 (Salmon et al., SC'11): the counter-based generator the sampler
    documents; ``counter`` four and ``key`` two 32-bit words."""
    c = list(counter)
    k = list(key)
    for _ in range(10):
        hi0, lo0 = _mulhilo(0xD2511F53, c[0])
        hi1, lo1 = _mulhilo(0xCD9E8D57, c[2])
        c = [hi1 ^ c[1] ^ k[0], lo1, hi0 ^ c[3] ^ k[1], lo0]
        k = [(k[0] + 0x9E3779B9) & 0xFFFFFFFF, (k[1] + 0xBB67AE85) & 0xFFFFFFFF]
    return c


def gumbel_noise(seed, stream, step, vocab):
    """Noise of the sampler for one row: token v uses word v % 4 of
    philox(counter=(v // 4, step, stream_lo, stream_hi), key=(seed_lo, seed_hi));
    u = ((word >> 9) + 0.5) * 2^-23 lies in (0, 1); the noise is -log(-log(u))."""
    out = np.empty(vocab, dtype=np.float64)
    key = (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    for base in range(0, vocab, 4):
        words = philox4x32((base // 4, step & 0xFFFFFFFF, stream & 0xFFFFFFFF,
                            (stream >> 32) & 0xFFFFFFFF), key)
        for j in range(min(4, vocab - base)):
            out[base + j] = ((words[j] >> 9) + 0.5) * 2.0 ** -23
    return -np.log(-np.log(out))


def sample_row(row, temperature, seed, stream, step):
    """serve.py:1544-1547 (Gumbel-max): argmax(logits / T + g); T == 0 means argmax."""
    if temperature == 0:
        return int(row.argmax())
    finite = row.double() / temperature
    noisy = finite.numpy() + gumbel_noise(seed, stream, step, row.shape[0])
    return int(np.argmax(noisy))
