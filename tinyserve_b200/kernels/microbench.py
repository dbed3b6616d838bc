"""Time one kernel of the package at a given size, after warm-up, with CUDA events.

    python -m tinyserve_b200.kernels.microbench gemm --m 8 --n 24576 --k 4096 [--splits S] [--impl tcgen05|cublas]
    python -m tinyserve_b200.kernels.microbench gemm --m 2048 --n 24576 --k 4096 --impl pair [--mode plain|gated|residual]
    python -m tinyserve_b200.kernels.microbench attention --batch 8 --q-len 1 --kv-len 640
    python -m tinyserve_b200.kernels.microbench norm --rows 8 --n 4096
    python -m tinyserve_b200.kernels.microbench rope --rows 2048

Every iteration uses another copy of the operands (``--copies``, sized so that together they
exceed the 126 MB L2), so the bytes really come from HBM.  ``--graph`` replays the loop from a
CUDA graph, as decode steps do.  Prints one JSON line with microseconds per call and the
achieved GB/s (algorithmic bytes / time) and TFLOP/s.  It is also the small case that the ncu
captures under profiles/ were taken on."""
from __future__ import annotations

import argparse
import json
from types import SimpleNamespace

import torch

from . import ops


def _time(fn, copies, iters, graph):
    for i in range(min(2, copies)):
        fn(i)
    torch.cuda.synchronize()
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(copies):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        if graph:
            g.replay()
        else:
            for i in range(copies):
                fn(i)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) * 1e3 / (iters * copies)


def bench_gemm(a):
    nbytes = a.n * a.k * 2
    copies = a.copies or max(2, min(16, int(300e6 // nbytes) + 1))
    ws = [torch.randn(a.n, a.k, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(a.m, a.k, device="cuda", dtype=torch.bfloat16)
    splits = a.splits or ops.gemm_splits(a.m, a.n, a.k)
    if a.impl.startswith("tcgen05"):
        fn = lambda i: ops._linear_tcgen05(x, ws[i], False, splits=splits, partials_only=a.partials_only)
    elif a.impl == "pair":
        # the paired kernel for many tokens, with the epilogue that the engine uses at this place
        res = torch.randn(a.m, a.n, device="cuda") if a.mode == "residual" else None
        wn = torch.ones(a.n, device="cuda", dtype=torch.bfloat16)
        if a.mode == "residual":
            fn = lambda i: ops._linear_pair(x, ws[i], residual=res, norm_weight=wn, pairs=a.pairs or None, halves=a.halves)
        else:
            fn = lambda i: ops._linear_pair(x, ws[i], gated=1 if a.mode == "gated" else 0, pairs=a.pairs or None, halves=a.halves)
    else:
        fn = lambda i: torch.mm(x, ws[i].t())
    us = _time(fn, copies, a.iters, a.graph)
    err = ops.gemm_tcgen05_error() if a.impl.startswith("tcgen05") else ops.gemm_pair_error() if a.impl == "pair" else 0
    return {"kernel": f"gemm_{a.impl}", "m": a.m, "n": a.n, "k": a.k, "splits": splits if a.impl.startswith("tcgen05") else None,
            "us": round(us, 2), "gbs": round((nbytes + a.m * (a.n + a.k) * 2) / us / 1e3, 1),
            "tflops": round(2.0 * a.m * a.n * a.k / us / 1e6, 2), "error_flag": err}


def bench_attention(a):
    H, Hkv, D, page = a.heads, a.kv_heads, a.head_dim, a.page
    B, q_len, kv_len = a.batch, a.q_len, a.kv_len
    pages_per = -(-kv_len // page)
    per_copy = B * pages_per
    copies = a.copies or max(2, min(16, int(300e6 // max(1, per_copy * 2 * Hkv * page * D * 2)) + 1))
    total_pages = per_copy * copies + 1
    kc = torch.randn(total_pages, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(total_pages, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
    tables = []
    for c in range(copies):
        perm = torch.randperm(per_copy) + 1 + c * per_copy
        tables.append(perm.view(B, pages_per).int().cuda())
    q = torch.randn(B * q_len, H, D, device="cuda", dtype=torch.bfloat16)
    cu = torch.arange(0, B * q_len + 1, q_len, dtype=torch.int32).cuda()
    kv = torch.full((B,), kv_len, dtype=torch.int32).cuda()
    # as the engine's step context: the lengths on the host too, and the work lists built once
    ctx = SimpleNamespace(cu_q=cu, kv_lens=kv, num_requests=B, max_q_len=q_len, max_kv_len=kv_len,
                          host={"cu_q": cu.tolist(), "kv_lens": kv.tolist()}, tile_cache={})
    views = [SimpleNamespace(block_table=t, page_size=page) for t in tables]
    fn = lambda i: ops.paged_attention(q, kc, vc, views[i], ctx, D ** -0.5, 0, num_splits=a.splits or None,
                                     backend=a.backend or None)
    us = _time(fn, copies, a.iters, a.graph)
    kv_bytes = B * kv_len * 2 * Hkv * D * 2
    flops = 4.0 * B * H * D * (q_len * kv_len - q_len * (q_len - 1) / 2)
    return {"kernel": "attention_decode" if q_len == 1 else "attention_prefill", "batch": B, "q_len": q_len,
            "kv_len": kv_len, "heads": H, "kv_heads": Hkv, "head_dim": D, "us": round(us, 2),
            "gbs": round(kv_bytes / us / 1e3, 1), "tflops": round(flops / us / 1e6, 2)}


def bench_norm(a):
    copies = a.copies or 4
    xs = [torch.randn(a.rows, a.n, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
    rs = [torch.randn(a.rows, a.n, device="cuda") for _ in range(copies)]
    w = torch.ones(a.n, device="cuda", dtype=torch.bfloat16)
    fn = lambda i: ops.add_rmsnorm(xs[i], rs[i], w, 1e-6, torch.bfloat16)
    us = _time(fn, copies, a.iters, a.graph)
    return {"kernel": "add_rmsnorm", "rows": a.rows, "n": a.n, "us": round(us, 2),
            "gbs": round(a.rows * a.n * 12 / us / 1e3, 1)}


def bench_rope(a):
    from ..parts.rotary import Rotary
    H, Hkv, D, page, T = a.heads, a.kv_heads, a.head_dim, a.page, a.rows
    copies = a.copies or 4
    qkvs = [torch.randn(T, (H + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
    pages = -(-T // page) + 1
    caches = [(torch.zeros(pages, Hkv, page, D, device="cuda", dtype=torch.bfloat16),
               torch.zeros(pages, Hkv, page, D, device="cuda", dtype=torch.bfloat16)) for _ in range(copies)]
    rot = Rotary(D, 1e6, "half")
    rot.cos, rot.sin = (t.cuda() for t in Rotary.tables(D, 1e6, max(T, 16)))
    pos = torch.arange(T, dtype=torch.int32).cuda()
    slots = torch.arange(page, page + T, dtype=torch.int32).cuda()
    qw = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    fn = lambda i: ops.qk_norm_rope_kvwrite(qkvs[i], pos, H, Hkv, D, rotary=rot, q_weight=qw, k_weight=qw, eps=1e-6,
                                            k_cache=caches[i][0], v_cache=caches[i][1], slot_mapping=slots,
                                            page_size=page)
    us = _time(fn, copies, a.iters, a.graph)
    return {"kernel": "qk_norm_rope_kvwrite", "rows": T, "heads": H, "kv_heads": Hkv, "head_dim": D,
            "us": round(us, 2), "gbs": round(T * (H + 2 * Hkv) * D * 4 / us / 1e3, 1)}


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m tinyserve_b200.kernels.microbench")
    ap.add_argument("kernel", choices=["gemm", "attention", "norm", "rope"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=24576)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--impl", choices=["tcgen05", "cublas", "pair"], default="tcgen05")
    ap.add_argument("--mode", choices=["plain", "gated", "residual"], default="plain", help="epilogue of --impl pair")
    ap.add_argument("--halves", type=int, default=0, help="--impl pair: tiles of 256 (1) or 512 (2) weight rows, 0: by estimate")
    ap.add_argument("--pairs", type=int, default=0, help="pairs of blocks of --impl pair (default: all the device holds)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--q-len", type=int, default=1)
    ap.add_argument("--kv-len", type=int, default=640)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--backend", choices=["tcgen05", "mma", "simt"], default="",
                    help="attention: a slower kernel than the one the head size selects")
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--copies", type=int, default=0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--graph", action="store_true")
    ap.add_argument("--partials-only", action="store_true",
                    help="gemm: stop after the split-K partial tiles (a consumer kernel adds them up)")
    a = ap.parse_args(argv)
    ops.require_device("cuda:0")
    out = {"gemm": bench_gemm, "attention": bench_attention, "norm": bench_norm, "rope": bench_rope}[a.kernel](a)
    out["graph"] = a.graph
    print(json.dumps(out))


if __name__ == "__main__":
    main()
