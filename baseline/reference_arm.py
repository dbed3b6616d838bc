"""The reference arm of bench.py: priyammaz/tinyserve itself, unmodified, on the same workload.

``serve.py``, ``tinykernels.py`` and ``tinycomm.py`` are plain Python files without a package
description, so the offline ``pip install`` has nothing to install; they are copied as they
are into ``baseline/_ref`` (not tracked) and imported from there.  This arm imports nothing
of tinyserve_b200.  It writes a model folder of the benchmark's shapes with random weights
(safetensors under the checkpoint's own tensor names, one file per layer) and a word-level
tokenizer of the right vocabulary built offline, then drives the reference's stock path:
``serve.Engine(serve.Config(...))`` with its defaults (Triton kernels and attention, CUDA
graphs, prefix caching), ``add_request(ids, SamplingParams)`` and ``step()``
(serve.py:2381-2447, 2449-2472, 2509-2601).

Measured like the repo's own arm: ``batch`` prompts of ``prompt_len`` random ids are
prefilled, ``warmup`` decode steps run untimed, then ``steps`` calls of ``Engine.step()`` are
timed with CUDA events (``value``) and with the wall clock, host ids in and sampled tokens out
(``e2e``); decode at batch 1 and 64 and one 2,048-token prompt are the ``points``.
"""
from __future__ import annotations

import json
import os
import shutil
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def _scratch_dir(need_bytes: int) -> str:
    """A temporary folder on the file system with the most room (the model folder is large)."""
    best, room = None, -1
    for cand in (os.environ.get("TMPDIR"), tempfile.gettempdir(), "/dev/shm", "/var/tmp"):
        if cand and os.path.isdir(cand) and os.access(cand, os.W_OK):
            free = shutil.disk_usage(cand).free
            if free > room:
                best, room = cand, free
    if best is None or room < need_bytes:
        raise RuntimeError(f"no temporary folder with {need_bytes / 2**30:.0f} GiB free "
                           f"(best: {best} with {max(room, 0) / 2**30:.0f} GiB)")
    return tempfile.mkdtemp(prefix="tinyserve_ref_", dir=best)


def write_model_folder(raw: dict, folder: str, seed: int) -> None:
    """config.json, tokenizer files and random weights under the checkpoint names that
    serve.load_model reads (serve.py:1289-1404): N(0, 0.02) matrices, norm weights
    1 + U(-0.1, 0.1), bfloat16, drawn on the device and written one file per layer."""
    import torch
    from safetensors.torch import save_file
    from tokenizers import Tokenizer, models, pre_tokenizers
    V, h, L = raw["vocab_size"], raw["hidden_size"], raw["num_hidden_layers"]
    H, Hkv, D, I = (raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"],
                    raw["intermediate_size"])
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(raw, fh)
    tok = Tokenizer(models.WordLevel(vocab={f"t{i}": i for i in range(V)}, unk_token="t0"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok.save(os.path.join(folder, "tokenizer.json"))
    with open(os.path.join(folder, "tokenizer_config.json"), "w") as fh:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "eos_token": "t1", "unk_token": "t0"}, fh)
    gen = torch.Generator(device="cuda").manual_seed(seed)

    def matrix(rows, cols):
        return (torch.randn(rows, cols, generator=gen, device="cuda") * 0.02).to(torch.bfloat16).cpu()

    def norm(n):
        return (1.0 + (torch.rand(n, generator=gen, device="cuda") * 0.2 - 0.1)).to(torch.bfloat16).cpu()

    save_file({"model.embed_tokens.weight": matrix(V, h), "model.norm.weight": norm(h)},
              os.path.join(folder, "model-embed.safetensors"))
    if not raw.get("tie_word_embeddings"):
        save_file({"lm_head.weight": matrix(V, h)}, os.path.join(folder, "model-head.safetensors"))
    for i in range(L):
        p = f"model.layers.{i}."
        save_file({
            p + "self_attn.q_proj.weight": matrix(H * D, h), p + "self_attn.k_proj.weight": matrix(Hkv * D, h),
            p + "self_attn.v_proj.weight": matrix(Hkv * D, h), p + "self_attn.o_proj.weight": matrix(h, H * D),
            p + "self_attn.q_norm.weight": norm(D), p + "self_attn.k_norm.weight": norm(D),
            p + "mlp.gate_proj.weight": matrix(I, h), p + "mlp.up_proj.weight": matrix(I, h),
            p + "mlp.down_proj.weight": matrix(h, I), p + "input_layernorm.weight": norm(h),
            p + "post_attention_layernorm.weight": norm(h)},
            os.path.join(folder, f"model-layer{i:03d}.safetensors"))


def _decode(serve, engine, batch, prompt_len, steps, warmup, vocab, seed, clock=None):
    import torch
    gen = torch.Generator().manual_seed(seed)
    params = serve.SamplingParams(temperature=0.0, max_tokens=warmup + steps + 8, repetition_penalty=1.0,
                                  ignore_eos=True)
    rids = [engine.add_request(torch.randint(0, vocab, (prompt_len,), generator=gen).tolist(), params)
            for _ in range(batch)]
    reqs = [engine.requests[r] for r in rids]
    guard = 0
    while any(len(r.output_ids) < 1 for r in reqs):
        engine.step()
        guard += 1
        if guard > 10000:
            raise RuntimeError("the reference engine did not finish the prompts")
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    if clock:
        clock.window(True)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    produced = 0
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        produced += len(engine.step())
    end.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    if clock:
        clock.window(False)
    ms = start.elapsed_time(end) / steps
    for r in rids:
        engine.abort(r)
    while engine.has_work():
        engine.step()
    return {"ms": ms, "tok_s": batch * 1000.0 / ms, "e2e": produced / wall}


def _prefill(serve, engine, tokens, vocab, seed, repeats=3):
    import torch
    gen = torch.Generator().manual_seed(seed)
    params = serve.SamplingParams(temperature=0.0, max_tokens=1, repetition_penalty=1.0, ignore_eos=True)
    times = []
    for _ in range(repeats + 1):
        ids = torch.randint(0, vocab, (tokens,), generator=gen).tolist()     # new ids: no cached prefix
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        engine.generate([ids], params)
        torch.cuda.synchronize()
        times.append((time.perf_counter() - t0) * 1000.0)
    return min(times[1:])


def burst(serve, raw: dict, seed: int) -> dict:
    """The reference's own burst workload (README.md:114-116) at Qwen3-0.6B shapes: 256 requests at
    once, prompts of 1 to 2,048 random tokens, 128 greedy tokens each, 2,048 tokens a step."""
    import torch
    V = raw["vocab_size"]
    folder = _scratch_dir(4 << 30)
    try:
        write_model_folder(raw, folder, seed)
        engine = serve.Engine(serve.Config(model=folder, max_model_len=4096, max_num_seqs=256,
                                           max_num_batched_tokens=2048))
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, 2049, (256,), generator=g).tolist()
    prompts = [torch.randint(0, V, (n,), generator=g).tolist() for n in lens]
    warm = serve.SamplingParams(temperature=0.0, max_tokens=4, repetition_penalty=1.0, ignore_eos=True)
    engine.generate([torch.randint(0, V, (64,), generator=g).tolist() for _ in range(8)], warm)
    params = serve.SamplingParams(temperature=0.0, max_tokens=128, repetition_penalty=1.0, ignore_eos=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate(prompts, params)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    generated = sum(len(o.token_ids) for o in outs)
    return {"burst_0p6b_total_tok_s": round((generated + sum(lens)) / dt, 1),
            "burst_0p6b_gen_tok_s": round(generated / dt, 1), "burst_0p6b_seconds": round(dt, 3)}


def long_context(serve, raw: dict, steps: int, warmup: int, seed: int) -> dict:
    """Decode at batch 8 with 4,096 and 16,384 tokens of context (the prompt fills it but for the
    decoded tokens), through an engine of its own with room for them."""
    V = raw["vocab_size"]
    h, L = raw["hidden_size"], raw["num_hidden_layers"]
    H, Hkv, D, I = (raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"], raw["intermediate_size"])
    weight_bytes = 2 * (L * ((H + 2 * Hkv) * D * h + h * H * D + 3 * I * h) + 2 * V * h)
    folder = _scratch_dir(int(weight_bytes * 1.05) + (1 << 30))
    try:
        write_model_folder(raw, folder, seed)
        engine = serve.Engine(serve.Config(model=folder, max_model_len=16384 + 256, max_num_seqs=8,
                                           max_num_batched_tokens=4096))
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    out = {}
    for name, ctx in (("decode_b8_ctx4k_tok_s", 4096), ("decode_b8_ctx16k_tok_s", 16384)):
        r = _decode(serve, engine, 8, ctx - warmup - steps - 8, steps, warmup, V, seed + ctx)
        out[name] = round(r["tok_s"], 1)
    return out


def run(raw: dict, batch: int, steps: int, warmup: int, seed: int, context: int, prompt_len: int,
        prefill_tokens: int, points: bool, peaks: dict, clock_sampler=None, burst_raw: dict = None) -> dict:
    """The reference's JSON line as a dict; raises if the reference cannot start."""
    if not os.path.isfile(os.path.join(REF, "serve.py")):
        raise RuntimeError("baseline/_ref/serve.py is not there (copy the reference's serve.py, "
                           "tinykernels.py and tinycomm.py into baseline/_ref)")
    assert not any(m == "tinyserve_b200" or m.startswith("tinyserve_b200.") for m in sys.modules), \
        "the reference arm must not load tinyserve_b200"
    if REF not in sys.path:
        sys.path.insert(0, REF)
    if clock_sampler:
        clock_sampler.start()
    import torch
    h, L, V = raw["hidden_size"], raw["num_hidden_layers"], raw["vocab_size"]
    H, Hkv, D, I = (raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"],
                    raw["intermediate_size"])
    weight_bytes = 2 * (L * ((H + 2 * Hkv) * D * h + h * H * D + 3 * I * h) + 2 * V * h)
    folder = _scratch_dir(int(weight_bytes * 1.05) + (1 << 30))
    try:
        t0 = time.time()
        write_model_folder(raw, folder, seed)
        print(f"[reference arm] model folder written in {time.time() - t0:.0f}s", file=sys.stderr, flush=True)
        import serve
        sizes = sorted({1, batch, 64}) if points else [batch]
        cfg = serve.Config(model=folder, max_model_len=context, max_num_seqs=max(sizes),
                           max_num_batched_tokens=prefill_tokens)
        engine = serve.Engine(cfg)
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    main = _decode(serve, engine, batch, prompt_len, steps, warmup, V, seed, clock_sampler)
    clocks = clock_sampler.stop() if clock_sampler else None
    line = {
        "metric": "decode tok/s (Qwen3-8B shapes, random weights)", "value": round(main["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
        "config": {"model": "Qwen3-8B shapes", "global_batch": batch, "seq_len": context,
                   "parallelism": "none", "layers": L, "layers_of_model": L, "hidden": h, "heads": H,
                   "kv_heads": Hkv, "head_dim": D, "intermediate": I, "vocab": V,
                   "prompt_len": prompt_len, "block_size": cfg.block_size,
                   "l2": "inputs larger than L2 (weights read every step)",
                   "attention_backend": cfg.attention_backend, "cuda_graphs": cfg.use_cuda_graphs},
        "clocks": clocks,
        "e2e": {"value": round(main["e2e"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": None, "d2h_bytes_per_step": batch * 8},
        "gpu_launches": None,
    }
    if points:
        pts = {}
        for b in (1, 64):
            r = _decode(serve, engine, b, prompt_len, min(steps, 64), warmup, V, seed + b)
            pts[f"decode_b{b}"] = round(r["tok_s"], 1)
        line["points"] = pts
        ms = _prefill(serve, engine, prefill_tokens, V, seed + 2)
        line["prefill"] = {"value": round(prefill_tokens * 1000.0 / ms, 1), "tokens": prefill_tokens,
                           "ms": round(ms, 3), "timed": "wall clock of Engine.generate, max_tokens 1"}
        if burst_raw is not None:
            import gc
            del engine
            gc.collect()
            torch.cuda.empty_cache()
            try:
                line["points"].update(burst(serve, burst_raw, seed))
            except Exception as exc:              # noqa: BLE001 - named in the line, the rest still prints
                line["points"]["burst_0p6b_error"] = f"{type(exc).__name__}: {exc}"[:200]
            gc.collect()
            torch.cuda.empty_cache()
            try:
                line["points"].update(long_context(serve, raw, min(steps, 32), warmup, seed))
            except Exception as exc:              # noqa: BLE001
                line["points"]["long_context_error"] = f"{type(exc).__name__}: {exc}"[:200]
    return line
