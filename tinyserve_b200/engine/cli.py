"""Command line in tinyserve's manner: ``python -m tinyserve_b200 generate --model DIR
--prompt "..."`` (serve.py:3098-3155).  Options that tinyserve has keep its names and
meanings; ``--dtype``, ``--block-size``, ``--num-blocks``, ``--prompt-ids``, ``--ignore-eos``,
``--top-p``, ``--top-k`` and the ``random-weights`` command are this engine's own.  The
``serve`` command (HTTP) is not part of this engine."""
from __future__ import annotations

import argparse
import json
import sys


def _ids(text: str) -> list:
    if text.startswith("@"):
        with open(text[1:]) as fh:
            text = fh.read()
    return [int(t) for t in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="tinyserve_b200")
    ap.add_argument("command", choices=["generate", "serve", "random-weights"])
    ap.add_argument("--model", required=False, help="model folder (config.json + safetensors)")
    ap.add_argument("--prompt", default="The capital of France is")
    ap.add_argument("--prompt-ids", type=_ids, default=None,
                    help="token ids instead of text: '1,2,3' or @file")
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=-1)
    ap.add_argument("--repetition-penalty", type=float, default=1.1,
                    help=">1 discourages repeating recent tokens, 1.0 = off")
    ap.add_argument("--repeat-last-n", type=int, default=64,
                    help="how many recent tokens the penalty looks at (0 = off, -1 = all)")
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--max-model-len", type=int, default=8192)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=2048)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.85)
    ap.add_argument("--no-cuda-graphs", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--block-size", type=int, default=0, help="tokens per cache page (0: 64 from 2,048 tokens of context on, else 16)")
    ap.add_argument("--num-blocks", type=int, default=0, help="cache pages per group (0: from memory)")
    # random-weights
    ap.add_argument("--config", help="random-weights: a config.json to make weights for")
    ap.add_argument("--out", help="random-weights: folder to write")
    ap.add_argument("--store-dtype", choices=["bfloat16", "float32"], default="bfloat16")
    return ap


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    if a.command == "serve":
        print("tinyserve_b200 has no HTTP server; use 'generate' or the Python entry point "
              "tinyserve_b200.LLM", file=sys.stderr)
        return 2
    if a.command == "random-weights":
        if not a.config or not a.out:
            print("random-weights needs --config and --out", file=sys.stderr)
            return 2
        from ..config.registry import config_from_dict
        from ..weights import write_random_model
        with open(a.config) as fh:
            config = config_from_dict(json.load(fh))
        write_random_model(config, a.out, seed=a.seed, store_dtype=a.store_dtype)
        print(a.out)
        return 0
    if not a.model:
        print("generate needs --model", file=sys.stderr)
        return 2
    from ..sampling import SamplingParams
    from .llm import LLM
    llm = LLM(a.model, dtype=a.dtype, max_model_len=a.max_model_len, max_num_seqs=a.max_num_seqs,
              max_num_batched_tokens=a.max_num_batched_tokens,
              gpu_memory_utilization=a.gpu_memory_utilization, use_cuda_graphs=not a.no_cuda_graphs,
              seed=a.seed, block_size=a.block_size, num_blocks=a.num_blocks, verbose=True)
    params = SamplingParams(temperature=a.temperature, top_p=a.top_p, top_k=a.top_k,
                            max_tokens=a.max_tokens, repetition_penalty=a.repetition_penalty,
                            repeat_last_n=a.repeat_last_n, ignore_eos=a.ignore_eos)
    prompt = a.prompt_ids if a.prompt_ids is not None else a.prompt
    out = llm.generate([prompt], params)[0]
    if a.prompt_ids is not None or llm.tokenizer is None:
        print(" ".join(str(t) for t in out.token_ids))
    else:
        print(a.prompt + out.text)
    return 0
