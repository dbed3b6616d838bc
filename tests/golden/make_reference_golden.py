"""Run priyammaz/tinyserve's own model code once, on the CPU in float32, on tiny random
Qwen3 models, and store its logits next to this script.

    python tests/golden/make_reference_golden.py --reference <checkout of priyammaz/tinyserve>

It imports the checkout's ``serve.py``, builds ``serve.Model`` (serve.py:1195), switches the
fused Triton ops off (``serve.TRITON_KERNELS = False``) and the attention to the plain
``serve.torch_ref_attention`` (serve.py:639), gives every layer a paged cache, loads the
weights of a folder written by ``write_random_model`` with q/k/v and gate/up fused as
``load_model`` does (serve.py:1352-1358), and runs ``Model.forward`` + ``Model.logits`` over a
prompt, whole and cut in two portions.  The weights are bfloat16 numbers (exact in the
reference's float32 model) and are stored beside the logits, as their 16-bit patterns, so that
``tests/test_plain.py`` holds the plain implementation to the stored logits with exactly the
tensors the reference ran on, whatever random numbers a torch version draws.
"""
import argparse
import importlib.util
import os
import sys
import tempfile
import types

import numpy as np
import torch
from safetensors.torch import load_file

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from helpers import make_model_dir, random_ids, tiny_config_dict  # noqa: E402

PROMPT_LEN = 37
BLOCK = 8


def reference_logits(serve, raw, tensors, ids, cuts):
    cfg = types.SimpleNamespace(**raw)
    serve.TRITON_KERNELS = False
    serve.ATTN_FN = serve.torch_ref_attention
    torch.set_default_dtype(torch.float32)
    model = serve.Model(cfg, max_position=64).eval()
    H, Hkv, D, I = (raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"],
                    raw["intermediate_size"])
    with torch.no_grad():
        params = dict(model.named_parameters())
        for name, t in tensors.items():
            name = name.removeprefix("model.")
            t = t.float()
            for part, (fused, lo, hi) in {
                    "q_proj": ("qkv_proj", 0, H * D), "k_proj": ("qkv_proj", H * D, (H + Hkv) * D),
                    "v_proj": ("qkv_proj", (H + Hkv) * D, (H + 2 * Hkv) * D),
                    "gate_proj": ("gate_up_proj", 0, I), "up_proj": ("gate_up_proj", I, 2 * I)}.items():
                if f".{part}." in name:
                    params[name.replace(part, fused)][lo:hi].copy_(t)
                    break
            else:
                params[name].copy_(t)
    nb = 64 // BLOCK + 1
    for layer in model.layers:
        layer.self_attn.kv_cache = torch.zeros(2, nb, BLOCK, Hkv, D)
    blocks = list(range(1, nb))
    out, start = [], 0
    with torch.no_grad():
        for n in cuts:
            pos = torch.arange(start, start + n)
            slots = torch.tensor([blocks[p // BLOCK] * BLOCK + p % BLOCK for p in pos.tolist()])
            serve.ATTN_META = serve.AttnMetadata(
                slot_mapping=slots, query_start_loc=torch.tensor([0, n], dtype=torch.int32),
                cu_seqlens_k=torch.tensor([0, start + n], dtype=torch.int32),
                block_table=torch.tensor([blocks], dtype=torch.int32), num_seqs=1, max_query_len=n,
                max_seq_len=start + n, query_start_loc_cpu=[0, n], seq_lens_cpu=[start + n])
            hidden = model(torch.tensor(ids[start:start + n]), pos)
            out.append(model.logits(hidden))
            start += n
    return torch.cat(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    a = ap.parse_args()
    spec = importlib.util.spec_from_file_location("serve", os.path.join(a.reference, "serve.py"))
    serve = importlib.util.module_from_spec(spec)
    sys.modules["serve"] = serve
    sys.path.insert(0, a.reference)
    spec.loader.exec_module(serve)
    for name in ("A", "B"):
        raw = tiny_config_dict(name)
        with tempfile.TemporaryDirectory() as folder:
            make_model_dir(folder, name, seed=11, store_dtype="bfloat16")
            tensors = load_file(os.path.join(folder, "model.safetensors"))
        ids = random_ids(raw["vocab_size"], PROMPT_LEN, seed=5)
        whole = reference_logits(serve, raw, tensors, ids, [PROMPT_LEN])
        cut = reference_logits(serve, raw, tensors, ids, [20, PROMPT_LEN - 20])
        print(name, "reference whole vs two portions:", (whole - cut).abs().max().item())
        stored = {"w:" + k: t.to(torch.bfloat16).view(torch.int16).numpy() for k, t in tensors.items()}
        np.savez_compressed(os.path.join(HERE, f"reference_logits_{name}.npz"), ids=np.array(ids),
                            logits=whole.numpy().astype(np.float32), **stored)
        print("wrote", f"reference_logits_{name}.npz", whole.shape)


if __name__ == "__main__":
    main()
