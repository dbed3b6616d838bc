"""When do the kernels of one decode step start, wait and finish?

    TINYSERVE_TIMELINE=1 python -m tinyserve_b200.kernels.timeline --layers 12 --batch 8 --prompt-len 512

The CUDA sources are built with TS_TIMELINE defined (build.py does that when TINYSERVE_TIMELINE=1):
thread 0 of every block then records the GPU's global timer when the block starts, when its wait
for the predecessor kernel returns, and at marks of the kernel's own.  This program runs a model of
the given layer sizes with random weights until every request decodes, records one decode step
(a CUDA graph replay, as in serving) and prints, for the kernels of two layers in the middle, the
times in microseconds from the first of them: when the first and the last block started, when the
first and the last wait returned, and the last mark 2 (a product's loads are all issued) and mark 3
(a product's results are stored).  A kernel's own time on the critical path is the span from its
last wait-return to the next kernel's; a product's loads run from before its wait (the first ring of
weight tiles does not depend on the predecessor) to mark 2.
"""
from __future__ import annotations

import argparse
import os
import sys


def collect(records):
    """Groups timeline records into launches, in time order.  A launch is a maximal set of blocks
    with the same grid and block size whose block indices are all different."""
    import numpy as np

    starts = records[records["tag"] == 0]
    launches = []
    for r in starts[np.argsort(starts["ns"], kind="stable")]:
        key = (tuple(int(v) for v in r["grid"]), int(r["threads"]))
        block = tuple(int(v) for v in r["block"])
        for launch in reversed(launches[-4:]):
            if launch["key"] == key and block not in launch["blocks"]:
                launch["blocks"].add(block)
                launch["start"].append(int(r["ns"]))
                break
        else:
            launches.append({"key": key, "blocks": {block}, "start": [int(r["ns"])], 1: [], 2: [], 3: []})
    for r in records[records["tag"] != 0]:
        key = (tuple(int(v) for v in r["grid"]), int(r["threads"]))
        owner = None
        for launch in launches:
            if launch["key"] == key and min(launch["start"]) <= int(r["ns"]):
                owner = launch
        if owner is not None and int(r["tag"]) in owner:
            owner[int(r["tag"])].append(int(r["ns"]))
    return launches


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--intermediate", type=int, default=12288)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--kernels", type=int, default=20, help="how many launches to print")
    ap.add_argument("--marks", action="store_true", help="also print the kernels' own marks of their traced blocks")
    a = ap.parse_args(argv)
    if os.environ.get("TINYSERVE_TIMELINE", "0") != "1":
        print("set TINYSERVE_TIMELINE=1: the kernels record nothing otherwise", file=sys.stderr)
        return 2

    import torch

    from .. import LLM, Qwen3Config, SamplingParams
    from . import ops

    raw = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", rms_norm_eps=1e-6, rope_theta=1e6,
               vocab_size=a.vocab, head_dim=a.head_dim, hidden_size=a.hidden, num_hidden_layers=a.layers,
               num_attention_heads=a.heads, num_key_value_heads=a.kv_heads, intermediate_size=a.intermediate,
               tie_word_embeddings=False)
    llm = LLM(model_config=Qwen3Config.from_dict(raw), random_weights=True, dtype="bfloat16",
              max_model_len=a.prompt_len + 256, block_size=16, max_num_seqs=a.batch,
              max_num_batched_tokens=max(4096, a.prompt_len), gpu_memory_utilization=0.5, verbose=False)
    gen = torch.Generator().manual_seed(0)
    params = SamplingParams(temperature=0.0, max_tokens=64, repetition_penalty=1.0, ignore_eos=True)
    for _ in range(a.batch):
        llm.add_request(torch.randint(0, a.vocab, (a.prompt_len,), generator=gen).tolist(), params)
    for _ in range(12):                  # prompts, then a few decode steps
        llm.step()
    torch.cuda.synchronize()
    ops.timeline_read(reset=True)
    llm.step()
    torch.cuda.synchronize()
    records = ops.timeline_read(reset=True)
    launches = collect(records)
    span = (int(records["ns"].max()) - int(records["ns"].min())) / 1e3
    print(f"{len(records)} records, {len(launches)} launches, step span {span:.1f} us")
    per_layer = max(1, (len(launches) - 3) // a.layers)
    first = min(len(launches) - 1, 1 + per_layer * (a.layers // 2))
    base = min(launches[first]["start"])

    def us(values, pick):
        return f"{(pick(values) - base) / 1e3:8.2f}" if values else "       -"

    print("grid x threads            blocks | first/last start | first/last wait return | loads issued | stored")
    for launch in launches[first:first + a.kernels]:
        grid, threads = launch["key"]
        print(f"{str(grid):>16} x {threads:<5} {len(launch['start']):5d} | {us(launch['start'], min)} {us(launch['start'], max)} |"
              f" {us(launch[1], min)} {us(launch[1], max)} | {us(launch[2], max)} | {us(launch[3], max)}")
    marks = records[records["tag"] >= 10]
    if a.marks and len(marks):
        # the kernels' own marks (one traced block or group of blocks per launch) inside the window shown
        t_lo, t_hi = base, max(max(launch["start"]) for launch in launches[first:first + a.kernels])
        print("marks of traced blocks (us, tag, value, grid):")
        for r in marks:
            if t_lo <= int(r["ns"]) <= t_hi + 20000:
                print(f"{(int(r['ns']) - base) / 1e3:8.2f}  tag {int(r['tag']):3d}  value {int(r['pad']):3d}  "
                      f"{tuple(int(v) for v in r['grid'])}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
