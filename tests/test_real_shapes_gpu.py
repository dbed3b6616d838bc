"""The step function at head sizes and widths that reach the fast kernels: the tcgen05 prefill
attention (head sizes 64 and 128), whole pages by TMA in decode (pages of 64), the tcgen05
products with their fused epilogues at 4,096 / 12,288 columns, and the three product paths that
the number of tokens selects (up to 16: fused layer, up to 64: tcgen05, above: the library).

Two configurations: the layer sizes of Qwen3-8B (two layers, a small vocabulary that is no
power of two) and a model of head size 64 with a group of three and widths that fill tiles
unevenly.  The per-head norm weights of q are scaled up so that the attention is peaked: a
wrong or missing key then moves the logits far beyond rounding.  The plain implementation runs
on the device in float64.

Two figures are held against a tolerance, both relative to the largest plain logit of the
request: the largest difference of any logit, and the largest root-mean-square difference over
the vocabulary at one position (a fault at one position moves that position's whole row, which
the second figure sees long before the first).  The tolerances are twice the largest values
measured on a B200; in bfloat16 the engine's error is about half of what the plain
implementation itself shows when torch runs it in bfloat16."""
import os

import numpy as np
import pytest
import torch
from safetensors.torch import load_file, save_file

import plain_qwen3 as plain
from helpers import (collect_logits, lines_of, max_live_tokens, random_ids, schedule_mixed,
                     schedule_portions, schedule_tail_decode, schedule_whole)

pytestmark = pytest.mark.gpu

CONFIGS = {
    "flagship_layers": dict(hidden_size=4096, num_hidden_layers=2, num_attention_heads=32,
                            num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=2003,
                            rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False),
    "head64_group3": dict(hidden_size=328, num_hidden_layers=3, num_attention_heads=6,
                          num_key_value_heads=2, head_dim=64, intermediate_size=576, vocab_size=1003,
                          rms_norm_eps=1e-5, rope_theta=1e4, tie_word_embeddings=True),
}
LENGTHS = {"flagship_layers": [300, 65, 17, 130, 520], "head64_group3": [410, 64, 3, 129, 777]}
# (largest difference, largest per-position rms difference) allowed, relative to the largest plain logit
# measured: float32 7.9e-6 / 1.8e-6 and 2.9e-6 / 7.0e-7; bfloat16 1.76e-2 / 4.1e-3 and 1.75e-2 / 4.7e-3
TOLERANCE = {("flagship_layers", "float32"): (1.6e-5, 3.7e-6), ("flagship_layers", "bfloat16"): (3.5e-2, 8.2e-3),
             ("head64_group3", "float32"): (6e-6, 1.4e-6), ("head64_group3", "bfloat16"): (3.5e-2, 9.4e-3)}
SHARPEN = 2.0


def errors(got, want, scale=None):
    """(largest difference, largest per-position rms difference) relative to ``scale`` (default: the
    largest |want|)."""
    diff = (got.double() - want).abs()
    scale = scale or want.abs().max().item()
    if diff.dim() == 1:
        diff = diff[None]
    return diff.max(-1).values / scale, diff.pow(2).mean(-1).sqrt() / scale


def make_folder(folder, name, seed):
    from tinyserve_b200.config import config_from_dict
    from tinyserve_b200.weights import write_random_model
    raw = dict(CONFIGS[name], architectures=["Qwen3ForCausalLM"], model_type="qwen3")
    write_random_model(config_from_dict(raw), str(folder), seed=seed, store_dtype="bfloat16")
    path = os.path.join(str(folder), "model.safetensors")
    tensors = load_file(path)
    for key in tensors:
        if key.endswith("q_norm.weight"):
            tensors[key] = (tensors[key].float() * SHARPEN).to(tensors[key].dtype)
    save_file(tensors, path, metadata={"format": "pt"})
    return str(folder)


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def model(request, tmp_path_factory):
    name = request.param
    folder = make_folder(tmp_path_factory.mktemp(name), name, seed=31)
    cfg, weights = plain.load_folder(folder)
    weights = {k: v.cuda() for k, v in weights.items()}
    reqs = {f"r{i}": random_ids(cfg["vocab_size"], n, seed=200 + i) for i, n in enumerate(LENGTHS[name])}
    with torch.no_grad():
        ref = {rid: plain.logits(cfg, weights, ids).cpu() for rid, ids in reqs.items()}
    return {"name": name, "folder": folder, "cfg": cfg, "weights": weights, "requests": reqs, "ref": ref}


def assert_no_kernel_gave_up(head_dim):
    from tinyserve_b200.kernels import ops
    assert ops.gemm_tcgen05_error() == 0
    assert ops.attention_tcgen05_error(head_dim) == 0
    assert ops.attention_mma_error(head_dim) == 0
    ops.raise_on_device_error()


def check(model, dtype, steps, out_dir, page, ref=None, max_live=8, graphs=False):
    from tinyserve_b200.engine import replay
    ref = ref or model["ref"]
    runner = replay.make_runner(model["folder"], dtype, max_live_tokens(steps, max(64, page)),
                                block_size=page, max_live=max_live, use_cuda_graphs=graphs)
    done = []
    replay.replay(runner, lines_of(steps), str(out_dir), done.append)
    assert len(done) == len(steps)
    runner.manager.check_invariants()
    assert not runner.manager.requests
    vocab = runner.model.vocab_size
    outputs = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        if wanted:
            outputs[s["step"]] = torch.from_numpy(np.fromfile(
                os.path.join(str(out_dir), f"{s['step']}.f32"), dtype="<f4").reshape(wanted, vocab))
    got = collect_logits(steps, outputs, vocab)
    worst_max = worst_rms = 0.0
    tol_max, tol_rms = TOLERANCE[(model["name"], dtype)]
    for rid, want in ref.items():
        if rid not in got:
            continue
        assert got[rid].shape == want.shape
        e_max, e_rms = errors(got[rid], want)
        bad = ((e_max > tol_max) | (e_rms > tol_rms)).nonzero()
        assert bad.numel() == 0, (f"{model['name']} {dtype} pages of {page}, request {rid}: first wrong token at "
                                  f"place {int(bad[0])} (largest {e_max[int(bad[0])]:.3e}, rms {e_rms[int(bad[0])]:.3e} "
                                  f"of the scale)")
        worst_max, worst_rms = max(worst_max, e_max.max().item()), max(worst_rms, e_rms.max().item())
    assert_no_kernel_gave_up(model["cfg"]["head_dim"])
    print(f"[measured] {model['name']} {dtype} page {page}: max {worst_max:.3e} rms {worst_rms:.3e}")
    if graphs:
        return runner
    return worst_max, worst_rms


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole(model, dtype, page, tmp_path):
    check(model, dtype, schedule_whole(model["requests"]), tmp_path, page)


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_32_tokens_one_by_one(model, dtype, page, tmp_path):
    check(model, dtype, schedule_tail_decode(model["requests"], 32), tmp_path, page)


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_changing_size(model, dtype, page, tmp_path):
    check(model, dtype, schedule_portions(model["requests"], sizes=(170, 9, 65, 3, 2, 128, 2, 31, 257)),
          tmp_path, page)
    short = {rid: ids for rid, ids in model["requests"].items() if len(ids) < 140}
    check(model, dtype, schedule_portions(short, sizes=(2,)), tmp_path / "twos", page,
          ref={rid: model["ref"][rid] for rid in short})


@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_with_pages_used_again(model, dtype, page, tmp_path):
    reqs = dict(model["requests"])
    more = {f"{rid}x": ids for rid, ids in reqs.items()}
    steps = schedule_mixed({**reqs, **more}, max_live=4, seed=1, chunk_sizes=(130, 2, 290, 61, 1))
    assert any(len({len(e["tokens"]) == 1 for e in s["entries"]}) == 2 for s in steps), \
        "portions stand beside decoded tokens"
    ref = {**model["ref"], **{f"{r}x": v for r, v in model["ref"].items()}}
    check(model, dtype, steps, tmp_path, page, ref=ref)
    total = sum(-(-len(i) // page) for i in {**reqs, **more}.values())
    assert total > max_live_tokens(steps, max(64, page)) // page, "the pool is too small to avoid reuse"


def test_products_of_many_tokens_on_the_paired_kernel(model, tmp_path, monkeypatch):
    """Every product of a step of more than 64 tokens on the paired tcgen05 kernel, with the
    residual add, the norm factor and the gated activation in the products' epilogues (the engine
    itself takes only the gate/up product of long prompts there): whole prompts and portions."""
    from tinyserve_b200.kernels import ops
    monkeypatch.setattr(ops, "PAIR_MIN_TOKENS", 65)
    monkeypatch.setattr(ops, "PAIR_GATED_MIN_TOKENS", 65)
    check(model, "bfloat16", schedule_whole(model["requests"]), tmp_path / "whole", 64)
    check(model, "bfloat16", schedule_portions(model["requests"], sizes=(170, 9, 65, 3, 2, 128, 2, 31, 257)),
          tmp_path / "portions", 16)
    assert ops.gemm_pair_error() == 0


def test_a_long_prompt_takes_the_paired_gate_up_product(model, tmp_path):
    """A prompt of 2,200 tokens at the layer sizes of Qwen3-8B, whole and in portions of 2,048 and
    152: the gate/up product of the long step runs on the paired tcgen05 kernel with the
    activation in its epilogue (what the engine does by itself from 2,048 tokens on), the short
    portion on the library's.  Both against the plain implementation."""
    if model["name"] != "flagship_layers":
        pytest.skip("the paired product takes rows of 4,096 elements and more")
    from tinyserve_b200.kernels import ops
    ids = random_ids(model["cfg"]["vocab_size"], 2200, seed=77)
    with torch.no_grad():
        ref = {"long": plain.logits(model["cfg"], model["weights"], ids).cpu()}
    reqs = {"long": ids}
    calls = []
    original = ops._linear_pair
    ops._linear_pair = lambda *a, **k: (calls.append(k.get("gated", 0)), original(*a, **k))[1]
    try:
        check(dict(model, requests=reqs), "bfloat16", schedule_whole(reqs), tmp_path / "whole", 64, ref=ref)
        assert calls and all(calls), "the long step's gate/up products ran on the paired kernel, gated"
        n = len(calls)
        check(dict(model, requests=reqs), "bfloat16", schedule_portions(reqs, sizes=(2048, 152)), tmp_path / "portions", 64, ref=ref)
        assert len(calls) == 2 * n, "the portion of 2,048 tokens too, the one of 152 not"
    finally:
        ops._linear_pair = original
    assert ops.gemm_pair_error() == 0


@pytest.mark.parametrize("page", [16, 64])
def test_steps_with_portions_replayed_from_graphs(model, page, tmp_path):
    """Steps of up to 512 tokens that hold prompt portions, padded to captured shapes and replayed
    from graphs (from the second time a shape comes up): the tcgen05 prefill kernel and the decode
    kernel run over work lists whose unused entries name an empty request."""
    reqs = dict(model["requests"])
    more = {f"{rid}x": ids for rid, ids in reqs.items()}
    ref = {**model["ref"], **{f"{r}x": v for r, v in model["ref"].items()}}
    steps = schedule_mixed({**reqs, **more}, max_live=4, seed=1, chunk_sizes=(130, 2, 290, 61, 1, 40, 130, 61))
    runner = check(model, "bfloat16", steps, tmp_path, page, ref=ref, graphs=True)
    assert runner.mixed_graph_replays > 0, "no step with portions was replayed from a graph"
    print(f"[measured] {model['name']} page {page}: {runner.mixed_graph_replays} of {len(steps)} steps replayed "
          f"from {sum(1 for v in runner.mixed_graphs.values() if not isinstance(v, int))} graphs of mixed steps")


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("page", [16, 64])
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_decode_batches_of_every_product_path(model, dtype, page, graphs, tmp_path):
    """1 to 72 live requests decode together: the fused layer (up to 16 tokens), the tcgen05
    products (up to 64) and the library products (above), from captured graphs and without."""
    from tinyserve_b200.config.engine_config import EngineConfig
    from tinyserve_b200.engine.batch import StepEntry
    from tinyserve_b200.engine.runner import ModelRunner
    if dtype == "float32" and (graphs or page == 64):
        pytest.skip("32-bit has one product path; one pass is enough")
    cfg, vocab = model["cfg"], model["cfg"]["vocab_size"]
    sizes, decode_steps, longest = (1, 8, 16, 17, 40, 64, 72), 3, 150
    g = torch.Generator().manual_seed(7)
    lengths = torch.randint(3, longest, (max(sizes),), generator=g).tolist()
    lengths[0], lengths[1] = longest, 1
    ids = [random_ids(vocab, n + decode_steps, seed=300 + i) for i, n in enumerate(lengths)]
    with torch.no_grad():
        ref = [plain.logits(cfg, model["weights"], seq).cpu() for seq in ids]
    ecfg = EngineConfig(model=model["folder"], dtype=dtype, max_model_len=256, block_size=page,
                        max_num_seqs=max(sizes), max_num_batched_tokens=2048, num_blocks=max(sizes) * (256 // page),
                        use_cuda_graphs=False)
    runner = ModelRunner(ecfg)
    if graphs:
        runner.capture_decode_graphs([1, 8, 16, 24, 40, 64, 72])
    tol_max, tol_rms = TOLERANCE[(model["name"], dtype)]
    worst_max = worst_rms = 0.0
    for n in sizes:
        rids = [f"d{n}_{i}" for i in range(n)]
        for rid in rids:
            runner.manager.begin(rid)
        # prompts in steps of up to 2,048 tokens
        at = 0
        while at < n:
            group, used = [], 0
            while at < n and used + lengths[at] <= 2048:
                group.append(at)
                used += lengths[at]
                at += 1
            logits = runner.step([StepEntry(rids[i], ids[i][:lengths[i]], [lengths[i] - 1]) for i in group])
            for row, i in enumerate(group):
                e_max, e_rms = errors(logits[row].cpu(), ref[i][lengths[i] - 1], ref[i].abs().max().item())
                assert e_max.item() <= tol_max and e_rms.item() <= tol_rms, f"prompt of request {i} in a batch of {n}"
        for t in range(decode_steps):
            entries = [StepEntry(rids[i], [ids[i][lengths[i] + t]], [0]) for i in range(n)]
            prep = runner.prepare(entries)
            assert (prep.graph is not None) == graphs
            logits = runner.launch(prep)
            rows = logits.cpu()
            for i in range(n):
                e_max, e_rms = errors(rows[i], ref[i][lengths[i] + t], ref[i].abs().max().item())
                assert e_max.item() <= tol_max and e_rms.item() <= tol_rms, (
                    f"{model['name']} {dtype}: request {i} of {n} (context {lengths[i] + t}), decode step {t}: "
                    f"largest {e_max.item():.3e}, rms {e_rms.item():.3e} of the scale")
                worst_max, worst_rms = max(worst_max, e_max.item()), max(worst_rms, e_rms.item())
        for rid in rids:
            runner.manager.free(rid)
    assert_no_kernel_gave_up(cfg["head_dim"])
    print(f"[measured] decode batches {model['name']} {dtype} page {page} graphs {graphs}: "
          f"max {worst_max:.3e} rms {worst_rms:.3e}")
