"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the
same ``ModelRunner.step`` (model, cache manager, kernels) that generation uses.  Steps come
as JSON lines: ``{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}],
"end": []}``.  For a step that wants logits, ``<out>/<step>.f32`` receives them as
little-endian float32 [wanted, vocab] in the order of the entries and of ``want``; after
every step a line ``done <step>`` is printed.  tinyserve has no such tool; its nearest
hooks are forced_token_ids and return_logprobs (serve.py:135-137, 2574-2579, 2659-2660).

The cache pool is made for ``--max-tokens`` tokens: the most that live requests hold at any
time, each request's count rounded up to a multiple of 64 (of the page size where pages are
larger), so that pages are used again.  ``--num-blocks`` sets the pool directly.
"""
from __future__ import annotations

import json
import os
import sys

DEFAULT_PAGE_SIZE = 16
DEFAULT_MAX_LIVE = 8
ROUND_TOKENS = 64


class TraceError(ValueError):
    """A step of the trace that the engine refuses before anything runs."""


def make_runner(model_dir: str, dtype: str, max_tokens: int, block_size: int = DEFAULT_PAGE_SIZE,
                max_live: int = DEFAULT_MAX_LIVE, num_blocks: int = 0, use_cuda_graphs: bool = False):
    from ..config.engine_config import EngineConfig
    from .runner import ModelRunner
    unit = max(ROUND_TOKENS, block_size)
    capacity = -(-max_tokens // unit) * unit
    cfg = EngineConfig(model=model_dir, dtype=dtype, max_model_len=capacity, block_size=block_size,
                       max_num_seqs=max_live, max_num_batched_tokens=capacity,
                       num_blocks=num_blocks or capacity // block_size, use_cuda_graphs=use_cuda_graphs)
    runner = ModelRunner(cfg)
    if use_cuda_graphs:
        runner.capture_decode_graphs()
    return runner


def _entries_of(record, runner):
    from .batch import StepEntry
    vocab = runner.model.vocab_size
    entries = []
    for e in record.get("entries", []):
        tokens = e.get("tokens")
        if not tokens:
            continue
        rid = e["id"]
        tokens = [int(t) for t in tokens]
        low, high = min(tokens), max(tokens)
        if low < 0 or high >= vocab:
            raise TraceError(f"step {record['step']}: request {rid!r} holds token id "
                             f"{low if low < 0 else high}, the vocabulary is [0, {vocab})")
        want = [int(j) for j in e.get("want", [])]
        if any(not 0 <= j < len(tokens) for j in want):
            raise TraceError(f"step {record['step']}: request {rid!r} wants a place outside its "
                             f"{len(tokens)} tokens")
        entries.append(StepEntry(rid, tokens, want))
    if len({e.rid for e in entries}) != len(entries):
        raise TraceError(f"step {record['step']}: a request appears twice")
    return entries


def replay(runner, lines, out_dir: str, report=print) -> int:
    os.makedirs(out_dir, exist_ok=True)
    steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = _entries_of(record, runner)
        for e in entries:
            if not runner.manager.is_live(e.rid):
                runner.manager.begin(e.rid)
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                data = logits.float().cpu().numpy().astype("<f4", copy=False)
                data.tofile(os.path.join(out_dir, f"{step}.f32"))
        for rid in record.get("end", []):
            if runner.manager.is_live(rid):
                runner.manager.free(rid)
        runner.raise_on_device_error()
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
    ap.add_argument("--block-size", type=int, default=DEFAULT_PAGE_SIZE, help="tokens per cache page")
    ap.add_argument("--max-live", type=int, default=DEFAULT_MAX_LIVE, help="most live requests")
    ap.add_argument("--num-blocks", type=int, default=0,
                    help="cache pages per group (default: --max-tokens worth of pages)")
    ap.add_argument("--cuda-graphs", action="store_true",
                    help="replay captured graphs for steps of single tokens, as serving does")
    args = ap.parse_args(argv)
    runner = make_runner(args.model, args.dtype, args.max_tokens, args.block_size, args.max_live,
                         args.num_blocks, args.cuda_graphs)

    def report(msg):
        sys.stdout.write(msg + "\n")
        sys.stdout.flush()

    replay(runner, sys.stdin, args.out, report)
    return 0
