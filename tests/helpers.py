"""Tiny configurations, model folders and replay schedules shared by the tests."""
from __future__ import annotations

import json

import torch

# Four tiny Qwen3 configurations that differ in every size and option.
TINY = {
    # MHA, head_dim * heads == hidden, tied embeddings
    "A": dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4,
              head_dim=16, intermediate_size=128, vocab_size=256, rms_norm_eps=1e-6, rope_theta=1e4,
              tie_word_embeddings=True, max_position_embeddings=128),
    # GQA 8/2, q projection wider than hidden, untied
    "B": dict(hidden_size=96, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2,
              head_dim=32, intermediate_size=160, vocab_size=384, rms_norm_eps=1e-5, rope_theta=1e6,
              tie_word_embeddings=False, max_position_embeddings=256),
    # sizes that are no power of two, group of 3, a window on the upper layers
    "C": dict(hidden_size=72, num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=2,
              head_dim=48, intermediate_size=100, vocab_size=301, rms_norm_eps=3e-6, rope_theta=5e5,
              tie_word_embeddings=False, max_position_embeddings=512, use_sliding_window=True,
              sliding_window=40, max_window_layers=2),
    # biases on q, k and v (drawn non-zero), widths that are multiples of 8 but fill no tile
    "D": dict(hidden_size=88, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, intermediate_size=136, vocab_size=211, rms_norm_eps=2e-6, rope_theta=2e5,
              tie_word_embeddings=False, max_position_embeddings=256, attention_bias=True),
}


def tiny_config_dict(name: str) -> dict:
    return dict(TINY[name], architectures=["Qwen3ForCausalLM"], model_type="qwen3")


def tiny_config(name: str):
    from tinyserve_b200.config import config_from_dict
    return config_from_dict(tiny_config_dict(name))


def make_model_dir(folder, name: str, seed: int = 0, store_dtype: str = "bfloat16",
                   vector_dtype=None) -> str:
    from tinyserve_b200.weights import write_random_model
    return write_random_model(tiny_config(name), str(folder), seed=seed, store_dtype=store_dtype,
                              vector_dtype=vector_dtype)


def random_ids(vocab: int, n: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ----------------------------------------------------------------------------- schedules
# A schedule is a list of steps {"step", "entries": [{"id", "tokens", "want"}], "end"}; every
# token's logits are wanted, so a replay yields the full [T, V] logits of every request.

def _step(i, entries, end=()):
    return {"step": i, "entries": entries, "end": list(end)}


def schedule_whole(requests: dict) -> list:
    """Each request alone and whole."""
    steps = []
    for rid, ids in requests.items():
        steps.append(_step(len(steps), [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], [rid]))
    return steps


def schedule_tail_decode(requests: dict, tail: int = 32) -> list:
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, ids in requests.items():
        head = max(1, len(ids) - tail)
        steps.append(_step(len(steps), [{"id": rid, "tokens": ids[:head], "want": list(range(head))}]))
        for t in range(head, len(ids)):
            steps.append(_step(len(steps), [{"id": rid, "tokens": [ids[t]], "want": [0]}],
                               [rid] if t == len(ids) - 1 else []))
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


def schedule_portions(requests: dict, sizes=(17, 9, 5, 3, 2, 2, 7, 2, 31, 4, 2)) -> list:
    """Portions of changing size, down to two tokens."""
    steps = []
    for rid, ids in requests.items():
        at, k = 0, 0
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            last = at + n == len(ids)
            steps.append(_step(len(steps), [{"id": rid, "tokens": ids[at:at + n], "want": list(range(n))}],
                               [rid] if last else []))
            at, k = at + n, k + 1
    return steps


def schedule_mixed(requests: dict, max_live: int = 4, seed: int = 0, chunk_sizes=(13, 2, 29, 6, 1)) -> list:
    """Up to ``max_live`` live requests; portions of some beside decoded tokens of others;
    a request may be left out of a step.  Requests start as earlier ones end, so that with a
    small pool their pages are used again."""
    g = torch.Generator().manual_seed(seed)
    waiting = list(requests.items())
    live, steps = {}, []          # rid -> [ids, at, decode_from]
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, ids = waiting.pop(0)
            # the last quarter of a request is fed token by token
            live[rid] = [ids, 0, max(1, len(ids) - max(2, len(ids) // 4))]
        entries, end = [], []
        for k, (rid, st) in enumerate(list(live.items())):
            ids, at, decode_from = st
            if len(live) > 1 and int(torch.randint(0, 5, (1,), generator=g)) == 0:
                continue                     # left out of this step
            if at >= decode_from:
                n = 1
            else:
                n = min(chunk_sizes[int(torch.randint(0, len(chunk_sizes), (1,), generator=g))],
                        decode_from - at)
            entries.append({"id": rid, "tokens": ids[at:at + n], "want": list(range(n))})
            st[1] = at + n
            if st[1] == len(ids):
                end.append(rid)
                del live[rid]
        if entries:
            steps.append(_step(len(steps), entries, end))
    return steps


def max_live_tokens(steps, round_to: int = 64) -> int:
    """Most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held, most = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return most


def collect_logits(steps, outputs: dict, vocab: int) -> dict:
    """{rid: [T, V] tensor} from per-step arrays ``outputs[step] -> [wanted, V]``."""
    rows = {}
    for s in steps:
        if not any(e["want"] for e in s["entries"]):
            continue
        data = outputs[s["step"]]
        k = 0
        for e in s["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(data[k])
                k += 1
        assert k == data.shape[0]
    return {rid: torch.stack(r) for rid, r in rows.items()}


def lines_of(steps) -> list:
    return [json.dumps(s) for s in steps]
