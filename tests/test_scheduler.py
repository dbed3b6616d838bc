"""The scheduler's decisions (no GPU), driven against the real cache manager with a step
function that only counts."""
import random

import pytest

from tinyserve_b200.cache import CacheManager, GroupSpec
from tinyserve_b200.engine.scheduler import Request, Scheduler
from tinyserve_b200.sampling import SamplingParams


def make(pages=64, page=8, seqs=4, budget=32):
    mgr = CacheManager([GroupSpec("full")], pages + 1, page, seqs)
    return Scheduler(mgr, seqs, budget), mgr


def req(rid, n, max_tokens=8):
    return Request(rid, list(range(n)), SamplingParams(max_tokens=max_tokens))


def run_step(sched, batch, finish_after=None):
    """What the engine does after a step: commit, append a token to whoever finished its prompt."""
    for s in batch:
        sched.manager.commit(s.req.request_id, s.num_new)
        if s.completes_prompt:
            s.req.token_ids.append(7)
            if len(s.req.output_ids) >= s.req.params.max_tokens:
                sched.finish(s.req, "length")


def test_budget_chunks_and_fifo():
    sched, mgr = make(budget=32)
    a, b, c = req("a", 40), req("b", 10), req("c", 5)
    for r in (a, b, c):
        sched.add(r)
    batch = sched.schedule()
    assert [(s.req.request_id, s.num_computed, s.num_new) for s in batch] == [("a", 0, 32)]
    assert not batch[0].completes_prompt
    run_step(sched, batch)
    batch = sched.schedule()
    # the running request first (rest of its prompt), then the queue in order, cut at the budget
    assert [(s.req.request_id, s.num_computed, s.num_new) for s in batch] == \
        [("a", 32, 8), ("b", 0, 10), ("c", 0, 5)]
    assert all(s.completes_prompt for s in batch)
    run_step(sched, batch)
    batch = sched.schedule()
    assert [(s.req.request_id, s.num_new) for s in batch] == [("a", 1), ("b", 1), ("c", 1)]


def test_max_num_seqs_and_head_of_line():
    sched, mgr = make(seqs=2, budget=64)
    for i, n in enumerate((4, 4, 4)):
        sched.add(req(f"r{i}", n, max_tokens=2))
    batch = sched.schedule()
    assert [s.req.request_id for s in batch] == ["r0", "r1"] and len(sched.waiting) == 1
    run_step(sched, batch)
    run_step(sched, sched.schedule())           # both reach max_tokens and leave
    assert [s.req.request_id for s in sched.schedule()] == ["r2"]


def test_preemption_takes_the_newest_and_recomputes():
    sched, mgr = make(pages=4, page=8, budget=64)     # 32 tokens of cache
    a, b = req("a", 15, max_tokens=20), req("b", 14, max_tokens=20)
    sched.add(a); sched.add(b)
    run_step(sched, sched.schedule())                  # 2 pages each, pool is full
    assert mgr.num_free_pages() == 0
    steps = 0
    while not b.was_preempted:
        run_step(sched, sched.schedule()); steps += 1
        assert steps < 10
    # a needed a third page; the newest request gave its pages back and waits at the front
    assert list(sched.waiting) == [b] and sched.running == [a]
    assert b.num_computed_tokens == 0 and not mgr.is_live("b")
    assert not a.was_preempted
    mgr.check_invariants()
    # nothing new is admitted in the step that preempted (serve.py:567)
    sched.finish(a, "length")
    batch = sched.schedule()
    assert [(s.req.request_id, s.num_computed, s.num_new) for s in batch] == [("b", 0, b.num_tokens)]
    assert b.num_tokens > 14, "the generated tokens are recomputed with the prompt"


def test_request_that_can_never_fit_ends_with_cache_full():
    sched, mgr = make(pages=2, page=8, budget=64)      # 16 tokens of cache
    a = req("a", 12, max_tokens=50)
    sched.add(a)
    for _ in range(20):
        batch = sched.schedule()
        if not batch:
            break
        run_step(sched, batch)
    assert a.finished and a.finish_reason == "cache_full" and sched.dropped == [a]
    assert not sched.has_work() and mgr.num_free_pages() == 2
    big = req("big", 40)
    sched.add(big)
    assert sched.schedule() == [] and big.finish_reason == "cache_full"
    mgr.check_invariants()


def test_abort_gives_pages_back():
    sched, mgr = make()
    a, b = req("a", 20), req("b", 3)
    sched.add(a); sched.add(b)
    run_step(sched, sched.schedule())
    sched.finish(a, "abort")
    assert a.finished and not mgr.is_live("a") and sched.running == [b]
    c = req("c", 3); sched.add(c); sched.finish(c, "abort")
    assert not sched.waiting
    mgr.check_invariants()


@pytest.mark.parametrize("seed", range(5))
def test_random_load_keeps_every_rule(seed):
    rng = random.Random(seed)
    budget, seqs = rng.choice([16, 32, 48]), rng.choice([2, 4, 6])
    sched, mgr = make(pages=rng.randint(10, 24), page=8, seqs=seqs, budget=budget)
    pending = [req(f"r{i}", rng.randint(1, 60), max_tokens=rng.randint(1, 12)) for i in range(25)]
    everyone = list(pending)
    for _ in range(3000):
        if pending and rng.random() < 0.3:
            sched.add(pending.pop(0))
        if not sched.has_work():
            if not pending:
                break
            continue
        batch = sched.schedule()
        assert sum(s.num_new for s in batch) <= budget
        assert len(batch) <= seqs and len(sched.running) <= seqs
        assert len({s.req.request_id for s in batch}) == len(batch)
        for s in batch:
            assert s.num_new >= 1 and s.num_computed == mgr.num_computed(s.req.request_id)
            assert s.num_computed + s.num_new <= s.req.num_tokens
        run_step(sched, batch)
        mgr.check_invariants()
    assert not sched.has_work() and not pending
    assert all(r.finished for r in everyone)
    assert all(p.num_free == p.num_usable for p in mgr.pools)


# ----------------------------------------------------------------------------- against tinyserve
def _reference_module():
    """tinyserve's own serve.py, unmodified, from baseline/_ref (not tracked); None if absent."""
    import importlib
    import os
    import sys
    ref = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
    if not os.path.isfile(os.path.join(ref, "serve.py")):
        return None
    if ref not in sys.path:
        sys.path.insert(0, ref)
    try:
        return importlib.import_module("serve")
    except Exception:           # an import of its dependencies that fails here
        return None


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_same_decisions_as_tinyserves_scheduler(seed):
    """The same arrivals given to tinyserve's Scheduler + KVCacheManager (serve.py:188-625, on the
    host, prefix cache off) and to this engine's: every step the same requests run with the same
    token counts from the same offsets, and the same requests are preempted."""
    serve = _reference_module()
    if serve is None:
        pytest.skip("tinyserve's serve.py is not under baseline/_ref (or does not import here)")
    from types import SimpleNamespace
    rng = random.Random(seed)
    pages, page, seqs, budget = rng.choice([(14, 8, 4, 32), (40, 16, 6, 64), (9, 4, 3, 16)])
    ours, _ = make(pages=pages, page=page, seqs=seqs, budget=budget)
    kv = serve.KVCacheManager(pages + 1, page, False)
    theirs = serve.Scheduler(SimpleNamespace(max_num_seqs=seqs, max_num_batched_tokens=budget, block_size=page), kv)
    longest = pages * page - 1                      # every request fits the pool when it is alone
    arrivals = []
    for i in range(30):
        n = rng.randint(1, min(longest - 12, 5 * budget))
        arrivals.append((rng.randint(0, 40), f"r{i}", n, rng.randint(1, 12)))
    arrivals.sort()
    mine, his = {}, {}
    step = 0
    preempted_mine, preempted_his = [], []
    while arrivals or ours.has_work() or theirs.has_work():
        while arrivals and arrivals[0][0] <= step:
            _, rid, n, max_tokens = arrivals.pop(0)
            mine[rid] = Request(rid, list(range(n)), SamplingParams(max_tokens=max_tokens))
            his[rid] = serve.Request(rid, list(range(n)), serve.SamplingParams(max_tokens=max_tokens))
            ours.add(mine[rid])
            theirs.add(his[rid])
        a, b = ours.schedule(), theirs.schedule()
        assert [(s.req.request_id, s.num_computed, s.num_new) for s in a] == \
               [(s.req.request_id, s.num_computed, s.num_new) for s in b], f"step {step}"
        assert [r.request_id for r in ours.running] == [r.request_id for r in theirs.running]
        assert [r.request_id for r in ours.waiting] == [r.request_id for r in theirs.waiting]
        preempted_mine.append(sorted(r for r, q in mine.items() if q.was_preempted))
        preempted_his.append(sorted(r for r, q in his.items() if q.was_preempted))
        run_step(ours, a)
        for s in b:                                 # what serve.Engine.step does with a batch
            if s.completes_prompt:
                s.req.token_ids.append(7)
                if len(s.req.output_ids) >= s.req.params.max_tokens:
                    theirs.finish(s.req, "length")
        assert not ours.dropped
        step += 1
        assert step < 5000
    assert preempted_mine == preempted_his
    assert any(preempted_mine[-1]) or pages > 30, "the small pools force preemption"
