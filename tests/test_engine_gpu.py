"""The entry point, the scheduler on the device, and each part alone."""
import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import make_model_dir, random_ids

pytestmark = pytest.mark.gpu


def llm_for(folder, dtype, **kw):
    from tinyserve_b200 import LLM
    opts = dict(dtype=dtype, max_model_len=256, block_size=16, max_num_seqs=8,
                max_num_batched_tokens=256, num_blocks=64, use_cuda_graphs=False)
    opts.update(kw)
    return LLM(folder, **opts)


def greedy(max_tokens):
    from tinyserve_b200 import SamplingParams
    return SamplingParams(temperature=0.0, max_tokens=max_tokens, repetition_penalty=1.0, ignore_eos=True)


def near_best(cfg, weights, prompt, out_ids, slack):
    """Every generated token is, under the plain logits of its own prefix, within ``slack``
    of the best token (bfloat16 may choose the other side of a near tie)."""
    ids = list(prompt)
    for tok in out_ids:
        row = plain.logits(cfg, weights, ids)[-1]
        assert row[tok] >= row.max() - slack * row.abs().max(), (len(ids), tok, int(row.argmax()))
        ids.append(tok)


def test_greedy_generation_tiny_a(tmp_path):
    """Three requests with prompts of 5, 17 and 31 tokens, 16 greedy tokens each."""
    folder = make_model_dir(tmp_path, "A", seed=31)
    cfg, weights = plain.load_folder(folder)
    prompts = [random_ids(256, n, seed=n) for n in (5, 17, 31)]
    outs = llm_for(folder, "float32").generate(prompts, greedy(16))
    for p, o in zip(prompts, outs):
        assert o.finished and o.finish_reason == "length" and o.num_prompt_tokens == len(p)
        assert o.token_ids == plain.greedy_generate(cfg, weights, p, 16)
    for graphs in (False, True):
        outs16 = llm_for(folder, "bfloat16", use_cuda_graphs=graphs).generate(prompts, greedy(16))
        for p, o in zip(prompts, outs16):
            assert len(o.token_ids) == 16
            near_best(cfg, weights, p, o.token_ids, 0.03)


def test_temperature_generation_tiny_b_with_chunked_prefill(tmp_path):
    """Five requests (1, 9, 40, 63, 100 tokens), 24 tokens at temperature 0.8, pages of 8, a
    budget of 32 tokens a step.  Every token is the arg-max of the plain logits / T plus the
    documented noise; the same tokens come out alone and in the batch."""
    from tinyserve_b200 import SamplingParams
    folder = make_model_dir(tmp_path, "B", seed=32)
    cfg, weights = plain.load_folder(folder)
    prompts = [random_ids(384, n, seed=n) for n in (1, 9, 40, 63, 100)]
    params = [SamplingParams(temperature=0.8, max_tokens=24, repetition_penalty=1.0, ignore_eos=True,
                             seed=1000 + i) for i in range(5)]
    kw = dict(block_size=8, max_num_batched_tokens=32, max_num_seqs=4, num_blocks=80, seed=7)
    outs = llm_for(folder, "float32", **kw).generate(prompts, params)
    assert any(o.was_chunked_prefill for o in outs)
    for i, (p, o) in enumerate(zip(prompts, outs)):
        ids = list(p)
        for step, tok in enumerate(o.token_ids):
            row = plain.logits(cfg, weights, ids)[-1]
            noisy = row.numpy() / 0.8 + plain.gumbel_noise(7, 1000 + i, step, 384)
            assert noisy[tok] >= noisy.max() - 1e-4, (i, step)
            ids.append(tok)
    alone = llm_for(folder, "float32", **kw).generate([prompts[3]], [params[3]])[0]
    assert alone.token_ids == outs[3].token_ids


@pytest.mark.parametrize("async_scheduling", [True, False])
def test_preemption_recomputes_the_same_tokens(tmp_path, async_scheduling):
    folder = make_model_dir(tmp_path, "A", seed=33)
    prompts = [random_ids(256, n, seed=n) for n in (30, 28, 26)]
    roomy = llm_for(folder, "float32", async_scheduling=False).generate(prompts, greedy(40))
    tight = llm_for(folder, "float32", num_blocks=9, async_scheduling=async_scheduling)   # 144 tokens for 3 x ~70
    outs = tight.generate(prompts, greedy(40))
    assert any(o.was_preempted for o in outs)
    assert [o.token_ids for o in outs] == [o.token_ids for o in roomy]
    tight.runner.manager.check_invariants()
    assert tight.runner.manager.num_free_pages() == 9


def test_many_requests_with_graphs_of_mixed_steps_under_preemption(tmp_path):
    """Eighty requests of 1 to 120 tokens through a pool too small for them, with 48 tokens a
    step: steps with prompt portions are padded to captured shapes and replayed from graphs,
    requests are pre-empted and recomputed, and every request still gets the tokens that the
    engine without graphs and with room for all gives it (32-bit, greedy)."""
    import random
    from tinyserve_b200 import SamplingParams
    folder = make_model_dir(tmp_path, "B", seed=5)
    rng = random.Random(1)
    prompts = [random_ids(384, rng.randint(1, 120), seed=i) for i in range(80)]
    params = [SamplingParams(temperature=0.0, max_tokens=rng.randint(1, 40), repetition_penalty=1.0, ignore_eos=True)
              for _ in prompts]
    kw = dict(max_model_len=192, block_size=8, max_num_seqs=12)
    roomy = llm_for(folder, "float32", async_scheduling=False, use_cuda_graphs=False, num_blocks=400,
                    max_num_batched_tokens=256, **kw).generate(prompts, params)
    tight = llm_for(folder, "float32", async_scheduling=True, use_cuda_graphs=True, num_blocks=60,
                    max_num_batched_tokens=48, **kw)
    outs = tight.generate(prompts, params)
    assert tight.runner.mixed_graph_replays > 20, "steps with portions were replayed from graphs"
    assert sum(o.was_preempted for o in outs) > 0
    assert [o.token_ids for o in outs] == [o.token_ids for o in roomy]
    tight.runner.manager.check_invariants()
    assert tight.runner.manager.num_free_pages() == 60


def test_a_capture_without_memory_turns_the_graphs_of_mixed_steps_off(tmp_path, monkeypatch):
    """A capture of a mixed step that runs out of memory leaves the engine as it was, with the
    feature off: the step runs eagerly, and so do all later ones."""
    folder = make_model_dir(tmp_path, "A", seed=33)
    prompts = [random_ids(256, n, seed=n) for n in (30, 28, 26, 31, 29, 27)]
    want = llm_for(folder, "float32", async_scheduling=False).generate(prompts, greedy(12))
    llm = llm_for(folder, "float32", use_cuda_graphs=True, max_num_batched_tokens=32, max_num_seqs=3)

    def no_memory(self, *args, **kwargs):
        raise torch.cuda.OutOfMemoryError("no memory for this capture (simulated)")

    monkeypatch.setattr(torch.cuda.CUDAGraph, "capture_begin", no_memory)
    assert llm.runner.mixed_graphs_enabled
    outs = llm.generate(prompts, greedy(12))
    assert not llm.runner.mixed_graphs_enabled and llm.runner.mixed_graph_replays == 0
    assert [o.token_ids for o in outs] == [o.token_ids for o in want]


def test_host_one_step_ahead_gives_the_same_tokens(tmp_path):
    """The loop that schedules step n+1 while step n runs (tokens fed back on the device) and the
    one-step-at-a-time loop produce the same tokens, with mixed sampling settings, chunked
    prompts, a stop token and graphs."""
    from tinyserve_b200 import SamplingParams
    folder = make_model_dir(tmp_path, "B", seed=35)
    prompts = [random_ids(384, n, seed=n) for n in (3, 50, 17, 90, 8, 33)]
    params = [SamplingParams(temperature=t, max_tokens=m, repetition_penalty=rp, top_k=k, top_p=p, seed=i)
              for i, (t, m, rp, k, p) in enumerate([(0.0, 30, 1.0, -1, 1.0), (0.8, 25, 1.0, -1, 1.0),
                                                     (0.0, 12, 1.3, -1, 1.0), (1.0, 40, 1.0, 20, 0.9),
                                                     (0.0, 1, 1.0, -1, 1.0), (0.7, 33, 1.1, -1, 0.95)])]
    results = []
    for async_scheduling, graphs in ((False, False), (True, False), (True, True)):
        llm = llm_for(folder, "float32", async_scheduling=async_scheduling, use_cuda_graphs=graphs,
                      max_num_batched_tokens=48, max_num_seqs=4, block_size=8, num_blocks=96)
        first = llm_for(folder, "float32", async_scheduling=False).generate([prompts[0]], greedy(5))[0].token_ids
        llm.stop_ids = {first[3]}             # request 0 stops at its fourth token
        outs = llm.generate(prompts, params)
        results.append([(o.token_ids, o.finish_reason) for o in outs])
        assert outs[0].finish_reason == "stop" and outs[0].token_ids == first[:4]
        assert not llm.has_work() and llm.runner.manager.num_free_pages() == 96
        llm.runner.manager.check_invariants()
    assert results[0] == results[1] == results[2]


def test_entry_point_options(tmp_path):
    from tinyserve_b200 import SamplingParams
    folder = make_model_dir(tmp_path, "A", seed=34)
    cfg, weights = plain.load_folder(folder)
    llm = llm_for(folder, "float32")
    p = random_ids(256, 12, seed=1)
    first = int(plain.logits(cfg, weights, p)[-1].argmax())
    # the stop id ends the request (no tokenizer here, so the engine is told the id)
    llm.stop_ids = {first}
    out = llm.generate([p], SamplingParams(temperature=0, max_tokens=5, repetition_penalty=1.0))[0]
    assert out.token_ids == [first] and out.finish_reason == "stop"
    llm.stop_ids = set()
    # forced tokens and the distributions that met them
    forced = [3, 4, 5]
    out = llm.generate([p], SamplingParams(temperature=0, max_tokens=3, repetition_penalty=1.0,
                                           forced_token_ids=forced, return_logprobs=True))[0]
    assert out.token_ids == forced and len(out.logprobs) == 3
    ref = torch.log_softmax(plain.logits(cfg, weights, p + forced[:2])[-1], -1)
    assert (out.logprobs[2].double() - ref).abs().max().item() < 1e-4
    # the repetition penalty changes the choice exactly as the plain formula says
    out = llm.generate([p], SamplingParams(temperature=0, max_tokens=2, repetition_penalty=50.0,
                                           repeat_last_n=-1, ignore_eos=True))[0]
    ids = list(p)
    for tok in out.token_ids:
        row = plain.repetition_penalty(plain.logits(cfg, weights, ids)[-1], ids, 50.0)
        assert tok == int(row.argmax())
        ids.append(tok)
    with pytest.raises(ValueError, match="tokenizer"):
        llm.add_request("text", greedy(1))
    with pytest.raises(ValueError, match="token id"):
        llm.add_request([1, 999], greedy(1))
    with pytest.raises(ValueError, match="max_model_len"):
        llm.add_request(list(range(200)) * 2, greedy(1))
    rid = llm.add_request(p, greedy(50))
    llm.step()
    llm.abort(rid)
    assert not llm.has_work() and llm.runner.manager.num_free_pages() == 64
    assert llm.stats()["generated_tokens"] > 0


def test_engine_fails_loudly_without_its_kernels(tmp_path, monkeypatch):
    from tinyserve_b200.kernels import build, ops
    monkeypatch.setattr(build, "_loaded", {})
    monkeypatch.setattr(build, "compile_unit", lambda *a, **k: str(tmp_path / "missing.so"))
    with pytest.raises(OSError):
        ops.embed_lookup(torch.zeros(4, 8, device="cuda"), torch.zeros(2, dtype=torch.int32, device="cuda"))
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.require_device("cpu")


# ----------------------------------------------------------------------------- parts alone
@pytest.fixture(scope="module")
def part_runner(tmp_path_factory):
    from tinyserve_b200.config import EngineConfig
    from tinyserve_b200.engine.runner import ModelRunner
    folder = make_model_dir(tmp_path_factory.mktemp("parts"), "C", seed=40, store_dtype="float32")
    runner = ModelRunner(EngineConfig(model=folder, dtype="float32", max_model_len=128, block_size=8,
                                      max_num_seqs=2, max_num_batched_tokens=128, num_blocks=32))
    cfg, weights = plain.load_folder(folder)
    return runner, cfg, weights


def _context(runner, n):
    from tinyserve_b200.engine.batch import StepEntry
    runner.manager.begin("x")
    ctx = runner._bind_device_views(runner._pack([StepEntry("x", [1] * n, [])]))
    runner._upload()
    return ctx


@pytest.mark.parametrize("layer", [0, 3])
def test_parts_alone(part_runner, layer):
    runner, cfg, w = part_runner
    T, hid = 50, cfg["hidden_size"]
    g = torch.Generator().manual_seed(layer)
    h = torch.randn(T, hid, generator=g)
    res = torch.randn(T, hid, generator=g)
    block = runner.model.blocks[layer]
    call = runner.model.calls[layer]
    ctx = _context(runner, T)
    try:
        p = f"model.layers.{layer}."
        cos, sin = plain.rope_tables(cfg["head_dim"], cfg["rope_theta"], T, torch.float64)
        window = plain.layer_window(cfg, layer)
        assert block.mixer.window == window == (40 if layer >= 2 else 0)
        # mixer
        got = block.mixer.forward(h.cuda(), ctx, call)
        want = plain.attention_block(h.double(), w, p + "self_attn.", cfg, cos, sin, window)
        assert (got.double().cpu() - want).abs().max().item() < 1e-5 * want.abs().max().item()
        # feed-forward
        got = block.ffn.forward(h.cuda(), ctx)
        want = plain.swiglu_mlp(h.double(), w, p + "mlp.")
        assert (got.double().cpu() - want).abs().max().item() < 1e-5 * want.abs().max().item()
        # norm with the residual sum
        r = res.clone().cuda()
        got = block.input_norm.add_forward(h.cuda(), r)
        want = plain.rms_norm(res.double() + h.double(), w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        assert (got.double().cpu() - want).abs().max().item() < 1e-5
        assert torch.equal(r.cpu(), res + h)
        # the block: x and residual in, next x out, residual advanced
        r = res.clone().cuda()
        x_next = block.forward(h.cuda(), r, ctx, call)
        full = plain.decoder_layer(res.double() + h.double(), w, layer, cfg, cos, sin, window)
        assert ((r.double() + x_next.double()).cpu() - full).abs().max().item() < 1e-5 * full.abs().max().item()
    finally:
        runner.manager.free("x")


def test_position_encoding_alone(part_runner):
    runner, cfg, _ = part_runner
    rot = runner.model.blocks[0].mixer.position
    cos, sin = plain.rope_tables(cfg["head_dim"], cfg["rope_theta"], 128, torch.float32)
    assert torch.equal(rot.cos.cpu(), cos) and torch.equal(rot.sin.cpu(), sin)
    assert rot.cos.data_ptr() == runner.model.blocks[3].mixer.position.cos.data_ptr(), "one table is shared"


def test_command_line_writes_random_weights_and_generates(tmp_path):
    """python -m tinyserve_b200 random-weights, then generate --prompt-ids: the command line drives
    the same engine and prints the same greedy tokens as the plain implementation."""
    import json
    import os
    import subprocess
    import sys
    from helpers import tiny_config
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(tiny_config("A").to_dict()))
    folder = str(tmp_path / "model")
    run = lambda *args: subprocess.run([sys.executable, "-m", "tinyserve_b200", *args], cwd=root,
                                       capture_output=True, text=True, timeout=600)
    made = run("random-weights", "--config", str(cfg_path), "--out", folder, "--seed", "7", "--store-dtype", "float32")
    assert made.returncode == 0 and made.stdout.strip() == folder, made.stderr
    prompt = random_ids(256, 9, seed=2)
    out = run("generate", "--model", folder, "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "10",
              "--temperature", "0", "--repetition-penalty", "1.0", "--ignore-eos", "--dtype", "float32",
              "--max-model-len", "64", "--max-num-seqs", "2", "--max-num-batched-tokens", "64",
              "--num-blocks", "16", "--no-cuda-graphs")
    assert out.returncode == 0, out.stderr[-2000:]
    cfg, weights = plain.load_folder(folder)
    assert [int(t) for t in out.stdout.strip().splitlines()[-1].split()] == plain.greedy_generate(cfg, weights, prompt, 10)
    assert run("serve").returncode == 2
    assert run("generate").returncode == 2


def test_host_index_check_refuses_a_corrupted_step(tmp_path):
    """The host half of the debug pass: a packed step whose index buffers do not fit the model,
    the batch or the cache is refused before it is uploaded."""
    from tinyserve_b200.config import EngineConfig
    from tinyserve_b200.engine.batch import StepEntry
    from tinyserve_b200.engine.runner import ModelRunner
    folder = make_model_dir(tmp_path, "A", seed=3)
    runner = ModelRunner(EngineConfig(model=folder, dtype="float32", max_model_len=64, block_size=16,
                                      max_num_seqs=2, max_num_batched_tokens=32, num_blocks=6))
    assert runner.cfg.check_indices, "tests run with the index check on"
    runner.manager.begin("a")
    entries = [StepEntry("a", [1, 2, 3], [2])]
    runner.step(entries)                                     # a sound step passes
    h = runner._hosts_np[0]
    for name, at, value, what in (("token_ids", 1, 256, "token id"), ("positions", 0, 64, "position"),
                                  ("logit_rows", 0, 3, "wanted row"), ("slot_mapping0", 2, 7 * 16, "cache slot"),
                                  ("pairs", 1, 7, "page number"), ("pairs", 0, 10 ** 6, "block-table change"),
                                  ("state_slots", 0, 3, "state slot"),
                                  ("cu_q", 1, 9, "query offsets")):
        ctx = runner._pack([StepEntry("a", [4, 5, 6], [2])], 0)
        runner._check_host(ctx, 0)
        if name == "pairs":
            h[runner._offsets["meta"][0]] = 1               # one block-table change: (index, page)
            h[runner._pairs_at + 1 - at], h[runner._pairs_at + at] = 1, value
        else:
            runner._seg(h, name)[at] = value
        with pytest.raises(ValueError, match=what):
            runner._check_host(ctx, 0)
    runner.manager.free("a")
