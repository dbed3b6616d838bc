"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the
same ``ModelRunner.step`` (model, cache manager, kernels) that generation uses.  Steps come
as JSON lines: ``{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}],
"end": []}``.  For a step that wants logits, ``<out>/<step>.f32`` receives them as
little-endian float32 [wanted, vocab] in the order of the entries and of ``want``; after
every step a line ``done <step>`` is printed.  tinyserve has no such tool; its nearest
hooks are forced_token_ids and return_logprobs (serve.py:135-137, 2574-2579, 2659-2660).
"""
from __future__ import annotations

import json
import os
import sys

PAGE_SIZE = 16
MAX_LIVE = 8


def make_runner(model_dir: str, dtype: str, max_tokens: int):
    from ..config.engine_config import EngineConfig
    from .runner import ModelRunner
    capacity = -(-max_tokens // 64) * 64
    cfg = EngineConfig(model=model_dir, dtype=dtype, max_model_len=capacity, block_size=PAGE_SIZE,
                       max_num_seqs=MAX_LIVE, max_num_batched_tokens=capacity,
                       num_blocks=capacity // PAGE_SIZE, use_cuda_graphs=False)
    return ModelRunner(cfg)


def replay(runner, lines, out_dir: str, report=print) -> int:
    from .batch import StepEntry
    os.makedirs(out_dir, exist_ok=True)
    steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = []
        for e in record.get("entries", []):
            if not e.get("tokens"):
                continue
            rid = e["id"]
            if not runner.manager.is_live(rid):
                runner.manager.begin(rid)
            entries.append(StepEntry(rid, list(e["tokens"]), list(e.get("want", []))))
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                data = logits.float().cpu().numpy().astype("<f4", copy=False)
                data.tofile(os.path.join(out_dir, f"{step}.f32"))
        for rid in record.get("end", []):
            if runner.manager.is_live(rid):
                runner.manager.free(rid)
        report(f"done {step}")
        steps += 1
    return steps


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time")
    args = ap.parse_args(argv)
    runner = make_runner(args.model, args.dtype, args.max_tokens)

    def report(msg):
        sys.stdout.write(msg + "\n")
        sys.stdout.flush()

    replay(runner, sys.stdin, args.out, report)
    return 0
