#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on Qwen3-8B shapes with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

A step is one decode step of the whole batch.  Prints ONE JSON line:
  value     decoded tokens per second over K steps, timed on the device with CUDA events;
            each step uploads the batch, runs the model and samples greedily on the device;
            tokens are fed back on the device and the host packs one step ahead
  e2e       the same through the Python entry point (LLM.add_request / LLM.step): host
            token ids in, sampled tokens out, scheduler and cache manager included
  prefill   one 2,048-token prompt in one step
  roofline  bytes the decode step must read (every weight once + the live cache) / time
  points    decode tokens per second at batch 1 and 64
The engine runs on one GPU; with --gpus > 1 it says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=4096,
                num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=12288, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6,
                tie_word_embeddings=False, max_position_embeddings=40960)
CONTEXT = 4096
PROMPT_LEN = 512
PREFILL_TOKENS = 2048
# the other two configurations of the baseline: a burst of short requests on a small model (it
# measures the host path and mixed batches) and a large model at long context
QWEN3_0P6B = dict(QWEN3_8B, hidden_size=1024, num_hidden_layers=28, num_attention_heads=16,
                  num_key_value_heads=8, intermediate_size=3072, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64,
                 num_key_value_heads=8, intermediate_size=25600)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi.  It runs from ``start()`` on (the
    tool needs a moment to come up, and the timed region may be shorter than that); ``window()``
    marks the timed region, and ``stop()`` reports the samples that fall into it (or, if the
    region was shorter than a sampling period, the samples nearest to it)."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.t0, self.t1 = [], None, None, None

    def start(self):
        if self.proc is not None:
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append((time.monotonic(), parts))

    def window(self, begin: bool):
        if begin:
            self.t0 = time.monotonic()
        else:
            self.t1 = time.monotonic()

    def stop(self):
        if self.proc is not None:
            time.sleep(0.12)                      # one more sample after the region
            self.proc.terminate()
        t0, t1 = self.t0 or 0.0, self.t1 or float("inf")
        inside = [s for t, s in self.samples if t0 <= t <= t1]
        if not inside and self.samples:
            mid = (t0 + min(t1, t0 + 3600)) / 2
            inside = [s for _, s in sorted(self.samples, key=lambda ts: abs(ts[0] - mid))[:3]]
        mhz = [int(s[0]) for s in inside if s[0].isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in inside)]
        mx = [int(s[1]) for s in inside if s[1].isdigit()]
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(inside)}


def decode_bytes(cfg, layers, batch, ctx):
    h, H, Hkv, D, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                          cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = ((H + 2 * Hkv) * D * h + h * H * D + 2 * I * h + h * I + 2 * h + 2 * D) * 2
    weights = layers * per_layer + V * h * 2 + h * 2
    kv = batch * ctx * layers * 2 * Hkv * D * 2
    return weights + kv


def prefill_flops(cfg, layers, T):
    h, H, Hkv, D, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                          cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    linear = 2 * T * layers * ((H + 2 * Hkv) * D * h + h * H * D + 3 * I * h) + 2 * V * h
    attention = layers * 4 * H * D * T * (T + 1) // 2
    return linear + attention


def run_decode(llm, batch, steps, warmup, seed, clock=None, prompt_len=PROMPT_LEN):
    """Prefill `batch` prompts of `prompt_len` tokens, then time `steps` decode steps."""
    import torch
    from tinyserve_b200.engine.batch import StepEntry
    from tinyserve_b200.kernels import ops
    runner, vocab = llm.runner, llm.runner.model.vocab_size
    gen = torch.Generator().manual_seed(seed)
    rids = [f"bench{batch}_{i}" for i in range(batch)]
    temps = torch.zeros(batch, dtype=torch.float32, device=runner.device)
    streams = torch.zeros(batch, dtype=torch.int64, device=runner.device)
    counters = torch.zeros(batch, dtype=torch.int32, device=runner.device)
    host = torch.empty(batch, dtype=torch.int32).pin_memory()
    last = []
    for rid in rids:
        runner.manager.begin(rid)
    budget = runner.cfg.max_num_batched_tokens
    if prompt_len <= budget:
        per_step = max(1, budget // prompt_len)
        for i in range(0, batch, per_step):
            group = rids[i:i + per_step]
            prompts = [torch.randint(0, vocab, (prompt_len,), generator=gen).tolist() for _ in group]
            logits = runner.step([StepEntry(r, p, [prompt_len - 1]) for r, p in zip(group, prompts)])
            last += logits.argmax(-1).tolist()
    else:
        for rid in rids:                      # a long prompt goes in portions of the budget
            ids = torch.randint(0, vocab, (prompt_len,), generator=gen).tolist()
            for at in range(0, prompt_len, budget):
                part = ids[at:at + budget]
                logits = runner.step([StepEntry(rid, part, [len(part) - 1] if at + budget >= prompt_len else [])])
            last += logits.argmax(-1).tolist()

    # Tokens stay on the device: the sampler leaves each request's token at its state slot and the
    # next step's embedding lookup reads it there.  The host packs step n+1 while step n runs and
    # never lags more than one step (it waits for the event of step n-1 before it reuses a buffer).
    from tinyserve_b200.engine.runner import PENDING
    slots = torch.tensor([runner.manager.slot(r) for r in rids], dtype=torch.int64, device=runner.device)
    runner.slot_tokens[slots] = torch.tensor(last, dtype=torch.int32, device=runner.device)
    entries = [StepEntry(r, [PENDING], [0]) for r in rids]
    events = []

    def one_step():
        if len(events) >= 2:
            events[-2].synchronize()
        logits = runner.step(entries)
        out = ops.sample(logits, temps, streams, counters, 0, slot_tokens=runner.slot_tokens,
                         slots=runner.state_slots_on_device(batch))
        host.copy_(out, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        events.append(ev)

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    if clock:
        clock.window(True)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ops.launch_count()
    start.record()
    for _ in range(steps):
        one_step()
    end.record()
    torch.cuda.synchronize()
    if clock:
        clock.window(False)
    clocks = clock.stop() if clock else None
    ms = start.elapsed_time(end) / steps
    ctx = prompt_len + warmup + steps / 2
    for rid in rids:
        runner.manager.free(rid)
    return {"ms": ms, "tok_s": batch * 1000.0 / ms, "ctx": ctx,
            "launches": ops.launch_count() - launches0, "clocks": clocks}


def run_e2e(llm, batch, steps, warmup, seed):
    """The same decode through LLM.add_request / LLM.step, wall clock, host ids in and out."""
    import torch
    from tinyserve_b200 import SamplingParams
    vocab = llm.runner.model.vocab_size
    gen = torch.Generator().manual_seed(seed + 1)
    params = SamplingParams(temperature=0.0, max_tokens=warmup + steps + 1, repetition_penalty=1.0,
                            ignore_eos=True)
    for i in range(batch):
        llm.add_request(torch.randint(0, vocab, (PROMPT_LEN,), generator=gen).tolist(), params,
                        request_id=f"e2e{i}")
    while any(r.num_computed_tokens < r.prompt_len for r in llm.requests.values()) or llm.scheduler.waiting:
        llm.step()
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += len(llm.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for rid in list(llm.requests):
        llm.abort(rid)
    h2d = llm.runner.last_upload_bytes
    return {"value": produced / dt, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": batch * 4}


def run_prefill(llm, seed, repeats=3):
    import torch
    from tinyserve_b200.engine.batch import StepEntry
    runner, vocab = llm.runner, llm.runner.model.vocab_size
    gen = torch.Generator().manual_seed(seed + 2)
    times = []
    for i in range(repeats + 1):
        rid = f"prefill{i}"
        runner.manager.begin(rid)
        ids = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepEntry(rid, ids, [PREFILL_TOKENS - 1])])
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
        runner.manager.free(rid)
    return min(times[1:])


def _release(llm):
    import gc
    import torch
    del llm
    gc.collect()
    torch.cuda.empty_cache()


def run_burst_0p6b(seed, block_size=16):
    """Qwen3-0.6B shapes: 256 requests arrive at once, prompts of 1 to 2,048 tokens, 128 greedy
    tokens each, 2,048 tokens a step, through LLM.generate.  Returns tokens per second (prompt +
    generated, and generated alone) over the whole run, wall clock."""
    import torch
    from tinyserve_b200 import LLM, Qwen3Config, SamplingParams
    llm = LLM(model_config=Qwen3Config.from_dict(QWEN3_0P6B), random_weights=True, dtype="bfloat16",
              max_model_len=4096, block_size=block_size, max_num_seqs=256, max_num_batched_tokens=2048, seed=seed)
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, 2049, (256,), generator=g).tolist()
    prompts = [torch.randint(0, QWEN3_0P6B["vocab_size"], (n,), generator=g).tolist() for n in lens]
    params = SamplingParams(temperature=0.0, max_tokens=128, repetition_penalty=1.0, ignore_eos=True)
    llm.generate(prompts[:8], SamplingParams(temperature=0.0, max_tokens=4, repetition_penalty=1.0, ignore_eos=True))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = llm.generate(prompts, params)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    generated = sum(len(o.token_ids) for o in outs)
    steps = llm.num_steps
    _release(llm)
    return {"burst_0p6b_total_tok_s": round((generated + sum(lens)) / dt, 1),
            "burst_0p6b_gen_tok_s": round(generated / dt, 1), "burst_0p6b_seconds": round(dt, 3),
            "burst_0p6b_steps": steps}


def run_large_32b(seed, block_size=16):
    """Qwen3-32B shapes at 8,192 context: 16 requests with prompts of 4,096 tokens and 256 greedy
    tokens each.  Returns prompt tokens per second while the prompts run and decoded tokens per
    second afterwards (CUDA events around the two phases, through LLM.step)."""
    import torch
    from tinyserve_b200 import LLM, Qwen3Config, SamplingParams
    llm = LLM(model_config=Qwen3Config.from_dict(QWEN3_32B), random_weights=True, dtype="bfloat16",
              max_model_len=8192, block_size=block_size, max_num_seqs=16, max_num_batched_tokens=4096,
              gpu_memory_utilization=0.9, seed=seed)        # the rest of the memory goes to the cache
    g = torch.Generator().manual_seed(seed)
    params = SamplingParams(temperature=0.0, max_tokens=256, repetition_penalty=1.0, ignore_eos=True)
    for i in range(16):
        llm.add_request(torch.randint(0, QWEN3_32B["vocab_size"], (4096,), generator=g).tolist(), params, request_id=f"big{i}")
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    torch.cuda.synchronize()
    marks[0].record()
    while any(r.num_computed_tokens < r.prompt_len for r in llm.requests.values()) or llm.scheduler.waiting:
        llm.step()
    marks[1].record()
    decoded = 0
    while llm.has_work():
        decoded += len(llm.step())
    marks[2].record()
    torch.cuda.synchronize()
    prefill_ms, decode_ms = marks[0].elapsed_time(marks[1]), marks[1].elapsed_time(marks[2])
    _release(llm)
    return {"large_32b_prefill_tok_s": round(16 * 4096 * 1000.0 / prefill_ms, 1),
            "large_32b_decode_b16_tok_s": round(decoded * 1000.0 / decode_ms, 1)}


def run_long_context(seed, steps, warmup, block_size=16):
    """Qwen3-8B shapes, batch 8, decode at 4,096 and at 16,384 tokens of context."""
    import torch
    from tinyserve_b200 import LLM, Qwen3Config
    from tinyserve_b200.engine.batch import StepEntry
    out = {}
    llm = LLM(model_config=Qwen3Config.from_dict(QWEN3_8B), random_weights=True, dtype="bfloat16",
              max_model_len=16384 + 256, block_size=block_size, max_num_seqs=8, max_num_batched_tokens=4096,
              num_blocks=8 * (16384 + 256) // block_size + 16, use_cuda_graphs=False, seed=seed)
    llm.runner.capture_decode_graphs([8])
    for name, ctx in (("decode_b8_ctx4k_tok_s", 4096), ("decode_b8_ctx16k_tok_s", 16384)):
        r = run_decode(llm, 8, steps, warmup, seed + ctx, prompt_len=ctx - warmup - steps)
        out[name] = round(r["tok_s"], 1)
    _release(llm)
    return out


def reference_main(a) -> int:
    """``--impl reference``: priyammaz/tinyserve, unmodified, from baseline/_ref, through its own
    Engine (see baseline/reference_arm.py).  If it cannot start here, the line says why."""
    if a.gpus != 1:
        print(f"bench.py: the reference arm runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm
        raw = dict(QWEN3_8B, num_hidden_layers=a.layers)
        line = reference_arm.run(raw, a.batch, a.steps, max(a.warmup, 3), a.seed, CONTEXT, PROMPT_LEN,
                                 PREFILL_TOKENS, not a.no_points, load_peaks(), ClockSampler(),
                                 burst_raw=None if a.no_workloads else QWEN3_0P6B)
    except BaseException as exc:                      # noqa: BLE001 - the reason goes into the line
        if isinstance(exc, KeyboardInterrupt):
            raise
        import traceback
        traceback.print_exc()
        why = f"{type(exc).__name__}: {exc}".replace("\n", " ")[:400]
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"])
    ap.add_argument("--impl", default="tinyserve_b200")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--block-size", type=int, default=64, help="tokens per cache page")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64 and prefill")
    ap.add_argument("--no-workloads", action="store_true",
                    help="skip the 0.6B burst, the 32B run and the long-context decode")
    a = ap.parse_args()
    if a.impl == "reference":
        return reference_main(a)
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    sampler = ClockSampler()
    sampler.start()                   # early: nvidia-smi takes longer to come up than a short timed region lasts
    import torch
    from tinyserve_b200 import LLM, Qwen3Config
    from tinyserve_b200.kernels import ops
    warmup = max(a.warmup, 3)
    raw = dict(QWEN3_8B, num_hidden_layers=a.layers)
    config = Qwen3Config.from_dict(raw)
    peaks = load_peaks()
    sizes = sorted({1, a.batch, 64}) if not a.no_points else [a.batch]
    llm = LLM(model_config=config, random_weights=True, dtype="bfloat16", max_model_len=CONTEXT,
              block_size=a.block_size, max_num_seqs=max(sizes), max_num_batched_tokens=PREFILL_TOKENS,
              num_blocks=max(sizes) * (CONTEXT // a.block_size) // 2 + 4096 // a.block_size, use_cuda_graphs=False,
              seed=a.seed)
    llm.runner.capture_decode_graphs(sizes)

    main_run = run_decode(llm, a.batch, a.steps, warmup, a.seed, sampler)
    e2e = run_e2e(llm, a.batch, a.steps, warmup, a.seed)
    points, prefill = {}, None
    if not a.no_points:
        for b in (1, 64):
            r = run_decode(llm, b, min(a.steps, 64), warmup, a.seed + b)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
        ms = run_prefill(llm, a.seed)
        flops = prefill_flops(raw, a.layers, PREFILL_TOKENS)
        prefill = {"value": round(PREFILL_TOKENS * 1000.0 / ms, 1), "tokens": PREFILL_TOKENS,
                   "ms": round(ms, 3), "frac": round(flops / (ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}
    if not a.no_points and not a.no_workloads and a.layers == QWEN3_8B["num_hidden_layers"]:
        _release(llm)
        llm = None
        for fn, args in ((run_burst_0p6b, (a.seed, a.block_size)), (run_large_32b, (a.seed, 16)),
                         (run_long_context, (a.seed, min(a.steps, 32), warmup, a.block_size))):
            try:
                points.update(fn(*args))
            except Exception as exc:                  # noqa: BLE001 - a workload that fails is named, the line still prints
                points[fn.__name__ + "_error"] = f"{type(exc).__name__}: {exc}"[:200]
    nbytes = decode_bytes(raw, a.layers, a.batch, main_run["ctx"])
    achieved = nbytes / (main_run["ms"] * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s (Qwen3-8B shapes, random weights)", "value": round(main_run["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": warmup,
        "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(main_run["tok_s"] / (42.2 * a.batch), 3) if a.batch == 1 else None,
        "dtype": "bf16", "data": "synthetic", "impl": "tinyserve_b200",
        "config": {"model": "Qwen3-8B shapes", "global_batch": a.batch, "seq_len": CONTEXT,
                   "parallelism": "none", "layers": a.layers,
                   "layers_of_model": QWEN3_8B["num_hidden_layers"], "hidden": raw["hidden_size"],
                   "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
                   "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"],
                   "vocab": raw["vocab_size"], "prompt_len": PROMPT_LEN, "block_size": a.block_size,
                   "l2": "inputs larger than L2 (weights read every step)",
                   "peaks": peaks["source"], "peak_hbm_gbs": peaks["hbm_gbs"],
                   "peak_bf16_tflops": peaks["bf16_tflops"]},
        "clocks": main_run["clocks"], "e2e": {k: (round(v, 1) if isinstance(v, float) else v)
                                               for k, v in e2e.items()},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4)},
    }
    if prefill:
        line["prefill"] = prefill
    if points:
        line["points"] = points
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
