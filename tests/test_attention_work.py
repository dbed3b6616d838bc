"""The work lists that a step's attention launches run from (kernels/ops.py: attention_work):
built on the host from the step's lengths, no GPU needed."""
import random
from types import SimpleNamespace

import torch

from tinyserve_b200.kernels import ops


def _ctx(q_lens, kv_lens):
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    return SimpleNamespace(num_requests=len(q_lens), host={"cu_q": cu, "kv_lens": list(kv_lens)},
                           cu_q=None, kv_lens=None, tile_cache={})


def test_portions_are_cut_into_blocks_and_one_token_requests_listed_apart():
    ctx = _ctx([1, 150, 1, 37, 2], [500, 150, 900, 437, 2])
    work = ops.attention_work(ctx, 64, torch.device("cpu"))
    blocks = list(zip(work.tile_req.tolist(), work.tile_q0.tolist()))
    assert sorted(blocks) == [(1, 0), (1, 64), (1, 128), (3, 0), (4, 0)]
    # heaviest first: the block whose first query sees the most keys
    seen = [ctx.host["kv_lens"][b] - (ctx.host["cu_q"][b + 1] - ctx.host["cu_q"][b]) + q0 for b, q0 in blocks]
    assert seen == sorted(seen, reverse=True)
    assert work.num_tiles == 5 and work.num_decode == 2
    assert work.dec_req.tolist() == [2, 0] and work.dec_tok.tolist() == [151, 0]      # longest context first
    assert work.max_decode_kv == 900
    assert ops.attention_work(ctx, 64, torch.device("cpu")) is work, "built once per step and block size"


def test_without_the_split_every_request_is_cut_into_blocks():
    ctx = _ctx([1, 5, 1], [9, 5, 1])
    work = ops.attention_work(ctx, 4, torch.device("cpu"), split_decodes=False)
    assert work.num_decode == 0
    assert sorted(zip(work.tile_req.tolist(), work.tile_q0.tolist())) == [(0, 0), (1, 0), (1, 4), (2, 0)]


def test_every_query_is_covered_once_under_random_lengths():
    rng = random.Random(3)
    for _ in range(50):
        q_lens = [rng.choice([1, 1, 2, rng.randint(1, 300)]) for _ in range(rng.randint(1, 12))]
        kv_lens = [n + rng.randint(0, 500) for n in q_lens]
        per = rng.choice([1, 2, 32, 64, 256])
        work = ops.attention_work(_ctx(q_lens, kv_lens), per, torch.device("cpu"))
        covered = {b: 0 for b in range(len(q_lens))}
        for b, q0 in zip(work.tile_req.tolist(), work.tile_q0.tolist()):
            assert q0 % per == 0 and q0 < q_lens[b]
            covered[b] += min(per, q_lens[b] - q0)
        for b in work.dec_req.tolist():
            assert q_lens[b] == 1
            covered[b] += 1
        assert all(covered[b] == q_lens[b] for b in covered)
