"""Trace replay against the plain implementation: each request alone and whole; most of it
in one step and the last 32 tokens one by one; portions of changing size down to two tokens;
mixed, up to four live requests with so few pages that they are used again; long decoding;
the first tokens of a sequence.  In 32-bit and in bfloat16, on three tiny configurations."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import (collect_logits, lines_of, make_model_dir, max_live_tokens, random_ids,
                     schedule_mixed, schedule_portions, schedule_tail_decode, schedule_whole, TINY)

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# Largest absolute logit difference allowed, relative to the largest plain logit.
# float32: rounding of 32-bit sums only (the plain side is float64).  bfloat16: activations
# carry 8 bits of mantissa (2^-8 = 0.4 %) through a few layers; per configuration, twice the
# largest value measured on a B200, and beside it the largest root-mean-square difference over
# the vocabulary at one position (a fault at one position moves its whole row).
# Measured (largest, rms): float32 5.2e-7, 1.3e-7 at most; bfloat16 A 2.7e-3, 8.5e-4;
# B 6.3e-3, 1.7e-3; C 6.3e-3, 1.8e-3; D 4.8e-3, 1.7e-3.
TOLERANCE = {"float32": 2e-6, "bfloat16": 1.3e-2}
BF16_TOLERANCE = {"A": (5.5e-3, 1.8e-3), "B": (1.3e-2, 3.5e-3), "C": (1.3e-2, 3.6e-3), "D": (1.0e-2, 3.5e-3)}
MEASURED = {}
LENGTHS = {"A": [5, 17, 31, 70, 2], "B": [1, 9, 40, 63, 100], "C": [90, 130, 57, 3, 75], "D": [33, 19, 80, 2, 64]}


@pytest.fixture(scope="module", params=sorted(TINY))
def model(request, tmp_path_factory):
    name = request.param
    folder = make_model_dir(tmp_path_factory.mktemp(f"tiny{name}"), name, seed=21,
                            vector_dtype="float32" if name == "B" else None)
    cfg, weights = plain.load_folder(folder)
    reqs = {f"r{i}": random_ids(cfg["vocab_size"], n, seed=100 + i) for i, n in enumerate(LENGTHS[name])}
    ref = {rid: plain.logits(cfg, weights, ids) for rid, ids in reqs.items()}
    return {"name": name, "folder": folder, "cfg": cfg, "weights": weights, "requests": reqs, "ref": ref}


def run_replay(folder, dtype, steps, out_dir, max_tokens=None, page=16, graphs=False):
    from tinyserve_b200.engine import replay
    runner = replay.make_runner(folder, dtype, max_tokens or max_live_tokens(steps), block_size=page,
                                use_cuda_graphs=graphs)
    done = []
    replay.replay(runner, lines_of(steps), str(out_dir), done.append)
    assert done == [f"done {s['step']}" for s in steps]
    runner.manager.check_invariants()
    assert not runner.manager.requests, "every request was ended"
    assert all(p.num_free == p.num_usable for p in runner.manager.pools), "every page came back"
    vocab = runner.model.vocab_size
    outputs = {}
    for s in steps:
        path = os.path.join(str(out_dir), f"{s['step']}.f32")
        wanted = sum(len(e["want"]) for e in s["entries"])
        assert os.path.isfile(path) == (wanted > 0)
        if wanted:
            outputs[s["step"]] = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(wanted, vocab))
    return outputs, runner


def check(model, dtype, steps, out_dir, max_tokens=None, page=16, graphs=False):
    outputs, runner = run_replay(model["folder"], dtype, steps, out_dir, max_tokens, page, graphs)
    got = collect_logits(steps, outputs, model["cfg"]["vocab_size"])
    worst = 0.0
    for rid, ref in model["ref"].items():
        if rid not in got:
            continue
        assert got[rid].shape == ref.shape
        err = (got[rid].double() - ref).abs().max(-1).values
        scale = ref.abs().max().item()
        tol_max, tol_rms = (TOLERANCE[dtype],) * 2 if dtype == "float32" else BF16_TOLERANCE[model["name"]]
        rms = (got[rid].double() - ref).pow(2).mean(-1).sqrt()
        bad = ((err > tol_max * scale) | (rms > tol_rms * scale)).nonzero()
        seen = MEASURED.setdefault((model["name"], dtype), [0.0, 0.0])
        seen[0], seen[1] = max(seen[0], err.max().item() / scale), max(seen[1], rms.max().item() / scale)
        assert bad.numel() == 0, (f"{model['name']} {dtype} request {rid}: first wrong token at place "
                                  f"{int(bad[0])} (error {err[int(bad[0])]:.3e}, scale {scale:.3e})")
        worst = max(worst, err.max().item() / scale)
    return worst, runner


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole(model, dtype, tmp_path):
    check(model, dtype, schedule_whole(model["requests"]), tmp_path)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_32_tokens_one_by_one(model, dtype, tmp_path):
    check(model, dtype, schedule_tail_decode(model["requests"], 32), tmp_path)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_changing_size(model, dtype, tmp_path):
    check(model, dtype, schedule_portions(model["requests"]), tmp_path)
    check(model, dtype, schedule_portions(model["requests"], sizes=(2,)), tmp_path / "twos")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [0, 1])
def test_mixed_with_pages_used_again(model, dtype, seed, tmp_path):
    reqs = dict(model["requests"])
    # the same five requests twice over, so that later ones get pages that earlier ones left
    cfg = model["cfg"]
    more = {f"{rid}x": ids for rid, ids in reqs.items()}
    steps = schedule_mixed({**reqs, **more}, max_live=4, seed=seed)
    assert max(len(s["entries"]) for s in steps) >= 3
    assert any(len({len(e["tokens"]) == 1 for e in s["entries"]}) == 2 for s in steps), \
        "portions stand beside decoded tokens"
    model = dict(model, ref={**model["ref"], **{f"{r}x": v for r, v in model["ref"].items()}})
    _, runner = check(model, dtype, steps, tmp_path)
    total = sum(-(-len(i) // 16) for i in {**reqs, **more}.values())
    assert total > runner.manager.pools[0].num_usable, "the pool is too small to avoid reuse"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_four_schedules_at_pages_of_8(model, dtype, tmp_path):
    """The page size of the second tiny configuration's workload: page edges fall elsewhere, a
    64-key tile of the attention kernels spans eight pages."""
    reqs = model["requests"]
    for name, steps in (("whole", schedule_whole(reqs)), ("tail", schedule_tail_decode(reqs, 32)),
                        ("portions", schedule_portions(reqs)), ("mixed", schedule_mixed(reqs, max_live=4, seed=2))):
        check(model, dtype, steps, tmp_path / name, page=8)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page", [16, 8])
def test_steps_with_portions_replayed_from_graphs(model, dtype, page, tmp_path):
    """With graphs on, a step that holds prompt portions is padded to a captured shape (tokens,
    requests, logit rows, context bound): the first step of a shape runs eagerly in the padded shape, the
    second is captured and replayed, later ones are replayed.  The logits stay those of the
    plain implementation: padding rows, empty requests and unused work-list entries change nothing."""
    reqs = dict(model["requests"])
    more = {f"{rid}x": ids for rid, ids in reqs.items()}
    both = dict(model, ref={**model["ref"], **{f"{r}x": v for r, v in model["ref"].items()}})
    replays = 0
    for seed in (0, 1):
        steps = schedule_mixed({**reqs, **more}, max_live=4, seed=seed)
        _, runner = check(both, dtype, steps, tmp_path / str(seed), page=page, graphs=True)
        assert runner.mixed_graphs_enabled
        replays += runner.mixed_graph_replays
        assert all(len(k) == 4 for k in runner.mixed_graphs)
    assert replays > 0, "no step with portions was replayed from a graph"


def test_a_bias_that_is_not_zero_reaches_the_logits(tmp_path):
    """The configuration with attention_bias draws its biases like matrices; without them the
    logits differ by far more than rounding, so a test that passes has used them."""
    folder = make_model_dir(tmp_path / "m", "D", seed=21)
    cfg, weights = plain.load_folder(folder)
    assert any(k.endswith("q_proj.bias") and v.abs().max() > 0 for k, v in weights.items())
    ids = random_ids(cfg["vocab_size"], 40, seed=1)
    with_bias = plain.logits(cfg, weights, ids)
    without = plain.logits(cfg, {k: v for k, v in weights.items() if not k.endswith(".bias")}, ids)
    assert (with_bias - without).abs().max().item() > 0.05 * with_bias.abs().max().item()


def test_schedules_agree_with_each_other_in_32_bit(model, tmp_path):
    """The logits at a position do not depend on how the tokens were cut."""
    reqs = model["requests"]
    a, _ = run_replay(model["folder"], "float32", schedule_whole(reqs), tmp_path / "a")
    steps_b = schedule_mixed(reqs, max_live=4, seed=3)
    b, _ = run_replay(model["folder"], "float32", steps_b, tmp_path / "b")
    whole = collect_logits(schedule_whole(reqs), a, 0)
    mixed = collect_logits(steps_b, b, 0)
    for rid in reqs:
        assert (whole[rid] - mixed[rid]).abs().max().item() < 2e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, tmp_path):
    """20 tokens at once, then 400 one by one: many page edges, and in configuration C the
    window passes pages that are given back while the request runs."""
    folder = make_model_dir(tmp_path / "m", "C", seed=5)
    cfg, weights = plain.load_folder(folder)
    ids = random_ids(cfg["vocab_size"], 420, seed=9)
    m = {"name": "C", "folder": folder, "cfg": cfg, "requests": {"long": ids},
         "ref": {"long": plain.logits(cfg, weights, ids)}}
    _, runner = check(m, dtype, schedule_tail_decode({"long": ids}, 400), tmp_path / "o")
    assert [g.kind for g in runner.manager.groups] == ["full", "window"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_one_by_one(model, dtype, tmp_path):
    ids = model["requests"]["r2"][:12]
    steps = [{"step": t, "entries": [{"id": "r2", "tokens": [ids[t]], "want": [0]}],
              "end": ["r2"] if t == 11 else []} for t in range(12)]
    m = dict(model, ref={"r2": model["ref"]["r2"][:12]})
    check(m, dtype, steps, tmp_path)


def test_steps_without_wanted_logits_and_skipped_requests(model, tmp_path):
    a, b = model["requests"]["r1"], model["requests"]["r2"]
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:4], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:7], "want": [6]}], "end": []},      # a is left out
        {"step": 2, "entries": [{"id": "b", "tokens": b[7:9], "want": []},
                                {"id": "a", "tokens": a[4:], "want": [len(a) - 5]}], "end": ["a", "b"]},
    ]
    out, _ = run_replay(model["folder"], "float32", steps, tmp_path, max_tokens=256)
    assert sorted(out) == [1, 2]
    scale = model["ref"]["r1"].abs().max().item()
    assert (out[1][0].double() - model["ref"]["r2"][6]).abs().max().item() < 2e-5 * scale
    assert (out[2][0].double() - model["ref"]["r1"][len(a) - 1]).abs().max().item() < 2e-5 * scale


def test_trace_run_program(tmp_path):
    """bin/trace_run as a program: stdin to files, 'done' lines, exit code 0."""
    folder = make_model_dir(tmp_path / "m", "B", seed=2)
    cfg, weights = plain.load_folder(folder)
    reqs = {"p": random_ids(cfg["vocab_size"], 45, seed=1), "q": random_ids(cfg["vocab_size"], 30, seed=2)}
    steps = schedule_mixed(reqs, max_live=2, seed=0)
    out = tmp_path / "out"
    for dtype in ("float32", "bfloat16"):
        proc = subprocess.run(
            [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
             "--out", str(out / dtype), "--max-tokens", str(max_live_tokens(steps))],
            input="\n".join(lines_of(steps)) + "\n", capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert proc.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
        outputs = {}
        for s in steps:
            wanted = sum(len(e["want"]) for e in s["entries"])
            outputs[s["step"]] = torch.from_numpy(np.fromfile(
                out / dtype / f"{s['step']}.f32", dtype="<f4").reshape(wanted, cfg["vocab_size"]))
        got = collect_logits(steps, outputs, cfg["vocab_size"])
        for rid, ids in reqs.items():
            ref = plain.logits(cfg, weights, ids)
            assert (got[rid].double() - ref).abs().max().item() < TOLERANCE[dtype] * ref.abs().max().item()


def test_zz_report_measured_errors():
    """Not a check: prints the largest errors that the tests above saw, per configuration and
    precision (with -s), the figures the bfloat16 tolerances are taken from."""
    for key in sorted(MEASURED):
        print(f"[measured] tiny {key[0]} {key[1]}: largest {MEASURED[key][0]:.3e}, per-position rms {MEASURED[key][1]:.3e}")
