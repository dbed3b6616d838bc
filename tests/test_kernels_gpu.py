"""Each CUDA kernel alone against a plain float64 reference written here, at sizes other
than the engine's tiny models use.  Inputs are made so that a fault shows: a far key that
dominates, a window's edge, pages in shuffled order."""
import math
from types import SimpleNamespace

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-5, torch.bfloat16: 8e-3}     # relative to the reference's scale; bfloat16: one rounding of the output (2^-9) and of each input


def ops():
    from tinyserve_b200.kernels import ops as o
    return o


def rnd(*shape, seed=0, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).cuda()


def close(got, want, dtype, what=""):
    want = want.double().cpu()
    err = (got.double().cpu() - want).abs().max().item()
    scale = max(want.abs().max().item(), 1e-6)
    assert err <= TOL[dtype] * scale, f"{what}: error {err:.3e} at scale {scale:.3e}"


# ----------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_lookup(dtype):
    table = rnd(301, 72, dtype=dtype)
    ids = torch.tensor([0, 300, 7, 7, 123], dtype=torch.int32).cuda()
    out = ops().embed_lookup(table, ids)
    assert out.dtype == torch.float32
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [72, 100, 1000, 1028, 4104, 8192])
@pytest.mark.parametrize("wdtype", ["same", "f32"])
def test_add_rmsnorm(dtype, n, wdtype):
    rows, eps = 7, 3e-6
    x = rnd(rows, n, seed=1, dtype=dtype)
    res = rnd(rows, n, seed=2, scale=3.0)
    w = rnd(n, seed=3, dtype=torch.float32 if wdtype == "f32" else dtype) + 1
    want_res = res.double() + x.double()
    want = want_res * torch.rsqrt(want_res.pow(2).mean(-1, keepdim=True) + eps) * w.double()
    r = res.clone()
    out = ops().add_rmsnorm(x, r, w, eps, dtype)
    close(out, want, dtype, "norm")
    assert (r.double() - want_res).abs().max().item() < 1e-6, "the residual sum is 32-bit"
    # without x: the residual is only normalised
    r2 = res.clone()
    out = ops().add_rmsnorm(None, r2, w, eps, dtype)
    v = res.double()
    close(out, v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.double(), dtype, "no add")
    assert torch.equal(r2, res)
    # gathered rows: only those rows, the residual untouched
    idx = torch.tensor([5, 0, 5], dtype=torch.int32).cuda()
    r3 = res.clone()
    out = ops().add_rmsnorm(x, r3, w, eps, dtype, rows=idx)
    close(out, want[idx.long().cpu()], dtype, "gather")
    assert torch.equal(r3, res)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_and_gated_activation(dtype):
    x = rnd(5, 3, 48, seed=4, dtype=dtype)
    w = rnd(48, seed=5, dtype=dtype)
    v = x.double()
    close(ops().rmsnorm(x, w, 1e-5), v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5) * w.double(),
          dtype, "rmsnorm")
    gu = rnd(9, 200, seed=6, dtype=dtype, scale=2.0)
    g, u = gu.double().chunk(2, -1)
    close(ops().gated_activation(gu, "silu"), g / (1 + torch.exp(-g)) * u, dtype, "silu")
    close(ops().gated_activation(gu, "gelu_tanh"),
          torch.nn.functional.gelu(g, approximate="tanh") * u, dtype, "gelu")
    # gate and up columns alternating in blocks (the layout of a row-interleaved fused weight)
    for block, inter in ((64, 192), (4, 100), (5, 15)):
        gb = rnd(7, 2 * inter, seed=7, dtype=dtype, scale=2.0)
        parts = gb.double().view(7, inter // block, 2, block)
        g, u = parts[:, :, 0].reshape(7, inter), parts[:, :, 1].reshape(7, inter)
        close(ops().gated_activation(gb, "silu", block=block), g / (1 + torch.exp(-g)) * u, dtype, f"blocks of {block}")


@pytest.mark.parametrize("M", [1, 8, 16, 40, 64])
@pytest.mark.parametrize("activation", ["silu", "gelu_tanh"])
def test_gated_product(M, activation):
    """The gate/up product with the activation in its epilogue (weight rows in blocks of 64), beside
    the same product followed by the activation kernel, from plain rows and from rows without
    their norm factor."""
    from tinyserve_b200.parts.base import interleave_halves
    o = ops()
    inter, K = 9600, 72           # 150 row tiles: the product needs no cut along K
    x = rnd(M, K, seed=1, dtype=torch.bfloat16)
    gate, up = rnd(inter, K, seed=2, dtype=torch.bfloat16, scale=0.3), rnd(inter, K, seed=3, dtype=torch.bfloat16, scale=0.3)
    w = interleave_halves(torch.cat([gate, up]), 64).contiguous()
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    act = (g / (1 + torch.exp(-g))) if activation == "silu" else torch.nn.functional.gelu(g, approximate="tanh")
    launches = o.launch_count()
    got = o.gated_linear(x, w, activation, 64)
    if M <= o.FUSED_MAX_TOKENS:
        assert o.launch_count() - launches == 1, "one kernel: the activation runs in the product's epilogue"
    assert got.shape == (M, inter)
    close(got, act * u, torch.bfloat16, "fused")
    # the kernel's gated form itself takes up to 64 tokens
    close(o._linear_tcgen05(x, w, False, splits=1, gated=o.ACTIVATIONS[activation] + 1), act * u, torch.bfloat16, "gated form")
    close(o.gated_activation(o.linear(x, w), activation, 64), act * u, torch.bfloat16, "product then activation")
    if M <= 16:
        sumsq = (rnd(1, 16, seed=5).abs() + 0.5).contiguous()
        rows = o.ScaledRows(x, sumsq, 1, 1e-6)
        scale = torch.rsqrt(sumsq[0, :M].double().cpu() / K + 1e-6)[:, None]
        gs, us = g.cpu() * scale, u.cpu() * scale
        acts = (gs / (1 + torch.exp(-gs))) if activation == "silu" else torch.nn.functional.gelu(gs, approximate="tanh")
        close(o.gated_linear(rows, w, activation, 64), acts * us, torch.bfloat16, "fused, scaled rows")
    assert o.gemm_tcgen05_error() == 0


def _rope_ref(x, pos, cos, sin, R, interleaved):
    xr, rest = x[..., :R], x[..., R:]
    c, s = cos[pos][:, None].double(), sin[pos][:, None].double()
    if interleaved:
        a, b = xr[..., 0::2], xr[..., 1::2]
        out = torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2)
    else:
        a, b = xr.chunk(2, -1)
        out = torch.cat([a * c - b * s, b * c + a * s], -1)
    return torch.cat([out, rest], -1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,Hkv,D,R,inter,norm,page", [
    (6, 3, 48, 48, False, True, 8), (8, 2, 128, 128, False, True, 16), (5, 5, 16, 16, False, False, 4),
    (4, 1, 80, 32, False, True, 16), (3, 3, 64, 64, True, True, 8), (2, 2, 96, 0, False, True, 16),
    (5, 2, 64, 64, False, True, 16), (3, 1, 256, 256, False, False, 8),
])
@pytest.mark.parametrize("T", [11, 300])        # few tokens: a warp per head; many: a block per token
def test_qk_norm_rope_kvwrite(dtype, H, Hkv, D, R, inter, norm, page, T):
    from tinyserve_b200.parts.rotary import Rotary
    pages, eps = -(-T // page) + 5, 1e-5
    qkv = rnd(T, (H + 2 * Hkv) * D, seed=7, dtype=dtype)
    pos = (torch.tensor([0, 1, 2, 30, 31, 32, 5, 6, 7, 63, 9] * (T // 11 + 1))[:T] +
           torch.arange(T) // 11 % 2).clamp(max=63).int().cuda()
    slots = torch.randperm(pages * page, generator=torch.Generator().manual_seed(3))[:T].int().cuda()
    slots[5] = -1                       # this token writes nothing
    rot = None
    if R:
        rot = Rotary(R, 1e4, "interleaved" if inter else "half")
        rot.cos, rot.sin = (t.cuda() for t in Rotary.tables(R, 1e4, 64))
    wdt = torch.float32 if D == 48 else dtype
    qw, kw = (rnd(D, seed=8, dtype=wdt) + 1, rnd(D, seed=9, dtype=wdt) + 1) if norm else (None, None)
    kc = torch.full((pages, Hkv, page, D), 7.0, dtype=dtype).cuda()
    vc = torch.full((pages, Hkv, page, D), 7.0, dtype=dtype).cuda()
    q = ops().qk_norm_rope_kvwrite(qkv, pos, H, Hkv, D, rotary=rot, q_weight=qw, k_weight=kw, eps=eps,
                                   k_cache=kc, v_cache=vc, slot_mapping=slots, page_size=page)
    x = qkv.double().cpu()
    qr, kr, vr = x.split([H * D, Hkv * D, Hkv * D], -1)
    qr, kr, vr = qr.view(T, H, D), kr.view(T, Hkv, D), vr.view(T, Hkv, D)
    if norm:
        n = lambda t, w: t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w.double().cpu()
        qr, kr = n(qr, qw), n(kr, kw)
    if R:
        p = pos.long().cpu()
        qr, kr = (_rope_ref(t, p, rot.cos.cpu(), rot.sin.cpu(), R, inter) for t in (qr, kr))
    close(q, qr, dtype, "q")
    want_k = torch.full((pages, Hkv, page, D), 7.0, dtype=torch.float64)
    want_v = want_k.clone()
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            want_k[s // page, :, s % page] = kr[t]
            want_v[s // page, :, s % page] = vr[t]
    close(kc, want_k, dtype, "k cache")
    assert torch.equal(vc.double().cpu(), want_v), "values are copied as they are"
    # no slots: only q, the cache stays
    kc2 = kc.clone()
    q2 = ops().qk_norm_rope_kvwrite(qkv, pos, H, Hkv, D, rotary=rot, q_weight=qw, k_weight=kw, eps=eps)
    assert torch.equal(q2, q) and torch.equal(kc2, kc)


# ----------------------------------------------------------------------------- matrix product
@pytest.mark.parametrize("M,N,K", [(5, 77, 50), (1, 301, 72), (70, 130, 52), (200, 96, 257), (33, 40, 8)])
@pytest.mark.parametrize("dtypes", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
def test_gemm_simt(M, N, K, dtypes):
    dtype, f32_out = dtypes
    o = ops()
    x, w, b = rnd(M, K, seed=1, dtype=dtype), rnd(N, K, seed=2, dtype=dtype), rnd(N, seed=3, dtype=dtype)
    linear = o.linear if dtype == torch.float32 else o._linear_simt
    out = linear(x, w, b, out_float32=f32_out)
    want = x.double() @ w.double().T + b.double()
    assert out.dtype == (torch.float32 if f32_out or dtype == torch.float32 else dtype)
    close(out, want, torch.float32 if f32_out else dtype, "gemm")
    # a row's result does not depend on the rows around it
    alone = linear(x[M // 2:M // 2 + 1].contiguous(), w, b, out_float32=f32_out)
    assert torch.equal(alone[0], out[M // 2])


def test_linear_bf16_library_path():
    x, w = rnd(9, 136, seed=1, dtype=torch.bfloat16), rnd(50, 136, seed=2, dtype=torch.bfloat16)
    out = ops().linear(x, w, out_float32=True)
    assert out.dtype == torch.float32
    close(out, x.double() @ w.double().T, torch.float32, "bf16 in, f32 out")
    close(ops().linear(x, w), x.double() @ w.double().T, torch.bfloat16, "bf16")


# ----------------------------------------------------------------------------- attention
def _paged(k, v, page, num_pages, seed):
    """Scatter per-request keys/values [n, Hkv, D] into shuffled pages.  Returns caches and a
    block table.  Unused slots hold large values, so that reading them shows."""
    Hkv, D = k[0].shape[1:]
    g = torch.Generator().manual_seed(seed)
    order = (torch.randperm(num_pages - 1, generator=g) + 1).tolist()
    kc = torch.full((num_pages, Hkv, page, D), 50.0, dtype=k[0].dtype)
    vc = torch.full((num_pages, Hkv, page, D), -50.0, dtype=k[0].dtype)
    max_blocks = max(-(-x.shape[0] // page) for x in k) + 2
    table = torch.zeros(len(k), max_blocks, dtype=torch.int32)
    for b, (kb, vb) in enumerate(zip(k, v)):
        for i in range(-(-kb.shape[0] // page)):
            pg = order.pop()
            table[b, i] = pg
            n = min(page, kb.shape[0] - i * page)
            kc[pg, :, :n] = kb[i * page:i * page + n].transpose(0, 1)
            vc[pg, :, :n] = vb[i * page:i * page + n].transpose(0, 1)
    return kc.cuda(), vc.cuda(), table.cuda()


def _attention_ref(q, k, v, q_lens, scale, window):
    """float64 reference: request b's last q_lens[b] positions attend to its keys."""
    out, at = [], 0
    for kb, vb, n in zip(k, v, q_lens):
        kv = kb.shape[0]
        qb = q[at:at + n].double()
        G = qb.shape[1] // kb.shape[1]
        kk, vv = kb.double().repeat_interleave(G, 1), vb.double().repeat_interleave(G, 1)
        s = torch.einsum("thd,shd->hts", qb, kk) * scale
        pos = torch.arange(kv - n, kv)
        j = torch.arange(kv)
        vis = j[None] <= pos[:, None]
        if window > 0:
            vis &= j[None] > pos[:, None] - window
        s = s.masked_fill(~vis[None], float("-inf"))
        out.append(torch.einsum("hts,shd->thd", s.softmax(-1), vv))
        at += n
    return torch.cat(out)


def _run_attention(q, kc, vc, table, q_lens, kv_lens, page, scale, window, splits, backend=None):
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32).cuda()
    ctx = SimpleNamespace(cu_q=cu, kv_lens=torch.tensor(kv_lens, dtype=torch.int32).cuda(),
                          num_requests=len(q_lens), max_q_len=max(q_lens), max_kv_len=max(kv_lens))
    view = SimpleNamespace(block_table=table, page_size=page)
    return ops().paged_attention(q, kc, vc, view, ctx, scale, window, num_splits=splits, backend=backend)


def _backends(dtype, D, page):
    """The kernels that can run this case: the one the engine picks by head size, and the slower
    ones below it (the engine reaches those at other head sizes)."""
    o = ops()
    chosen = o.attention_backend(dtype, D, page)
    return {"tcgen05": ["tcgen05", "mma", "simt"], "mma": ["mma", "simt"], "simt": ["simt"]}[chosen]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,Hkv,D,page", [(6, 2, 48, 8), (4, 4, 16, 16), (8, 1, 64, 4), (40, 1, 32, 16),
                                           (5, 5, 80, 32), (16, 2, 128, 16), (80, 1, 16, 8), (4, 2, 256, 16),
                                           (32, 8, 128, 16), (6, 2, 64, 8), (3, 1, 128, 128), (200, 1, 64, 16)])
@pytest.mark.parametrize("window,splits", [(0, 1), (0, 3), (23, 1), (23, 4)])
def test_paged_attention_mixed_batch(dtype, H, Hkv, D, page, window, splits):
    # a whole prompt, a decode token, a portion after a prefix, two tokens, a long decode
    kv_lens, q_lens = [70, 133, 97, 2, 300], [70, 1, 29, 2, 1]
    k = [rnd(n, Hkv, D, seed=10 + i, dtype=dtype).cpu() for i, n in enumerate(kv_lens)]
    v = [rnd(n, Hkv, D, seed=20 + i, dtype=dtype).cpu() for i, n in enumerate(kv_lens)]
    q = rnd(sum(q_lens), H, D, seed=30, dtype=dtype)
    kc, vc, table = _paged(k, v, page, sum(-(-n // page) for n in kv_lens) + 3, seed=1)
    want = _attention_ref(q.cpu(), k, v, q_lens, D ** -0.5, window)
    for backend in _backends(dtype, D, page):
        if backend == "tcgen05" and splits > 1:
            continue                       # prefill has no key ranges
        out = _run_attention(q, kc, vc, table, q_lens, kv_lens, page, D ** -0.5, window, splits, backend)
        close(out, want, dtype, f"attention ({backend})")
    if dtype == torch.bfloat16 and D in ops().TCGEN05_HEAD_DIMS:
        assert ops().attention_tcgen05_error(D) == 0


@pytest.mark.parametrize("H,Hkv,D,page", [(16, 8, 128, 16), (6, 2, 64, 8), (10, 2, 48, 16)])
@pytest.mark.parametrize("window", [0, 200])
def test_paged_attention_many_decodes_beside_portions(H, Hkv, D, page, window):
    """A serving step in the middle of a run: many requests decode, two bring portions of their
    prompts.  The one-token requests go to the decode kernel by a request list (long ones in
    several key ranges), the portions to the prefill kernel by a work list of blocks."""
    dtype = torch.bfloat16
    gen = torch.Generator().manual_seed(5)
    q_lens = [1, 1, 150, 1, 1, 1, 37, 1, 1, 2, 1]
    kv_lens = [int(torch.randint(1, 900, (1,), generator=gen)) + n for n in q_lens]
    kv_lens[3], kv_lens[7] = 1, 1500         # a first token; a context long enough for key ranges
    k = [rnd(n, Hkv, D, seed=40 + i, dtype=dtype).cpu() for i, n in enumerate(kv_lens)]
    v = [rnd(n, Hkv, D, seed=60 + i, dtype=dtype).cpu() for i, n in enumerate(kv_lens)]
    q = rnd(sum(q_lens), H, D, seed=31, dtype=dtype)
    kc, vc, table = _paged(k, v, page, sum(-(-n // page) for n in kv_lens) + 5, seed=2)
    want = _attention_ref(q.cpu(), k, v, q_lens, D ** -0.5, window)
    for backend in _backends(dtype, D, page):
        out = _run_attention(q, kc, vc, table, q_lens, kv_lens, page, D ** -0.5, window, None, backend)
        close(out, want, dtype, f"attention ({backend})")
    if D in ops().TCGEN05_HEAD_DIMS:
        assert ops().attention_tcgen05_error(D) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,Hkv,D,page", [(4, 4, 64, 16), (8, 2, 128, 16), (20, 1, 48, 8), (3, 1, 256, 32),
                                           (8, 2, 128, 64), (6, 3, 64, 32)])      # pages of 32 and 64: whole pages by TMA
@pytest.mark.parametrize("window,splits", [(0, 1), (0, 7), (130, 1), (130, 3), (0, 11)])   # 11 ranges: no cluster
def test_paged_attention_decode_batch(dtype, H, Hkv, D, page, window, splits):
    """Every request brings one token: the decode kernels."""
    kv_lens = [1, 64, 65, 300, 129, 1000, 17]
    q_lens = [1] * len(kv_lens)
    k = [rnd(n, Hkv, D, seed=10 + i, dtype=dtype).cpu() for i, n in enumerate(kv_lens)]
    v = [rnd(n, Hkv, D, seed=20 + i, dtype=dtype).cpu() for i, n in enumerate(kv_lens)]
    q = rnd(len(kv_lens), H, D, seed=30, dtype=dtype)
    kc, vc, table = _paged(k, v, page, sum(-(-n // page) for n in kv_lens) + 3, seed=4)
    want = _attention_ref(q.cpu(), k, v, q_lens, D ** -0.5, window)
    for backend in _backends(dtype, D, page):
        if backend == "tcgen05":
            continue                       # decode has no tcgen05 kernel: it is the mma decode kernel
        out = _run_attention(q, kc, vc, table, q_lens, kv_lens, page, D ** -0.5, window, splits, backend)
        close(out, want, dtype, f"decode attention ({backend})")
    if dtype == torch.bfloat16 and D <= ops().MMA_MAX_HEAD_DIM:
        assert ops().attention_mma_error(D) == 0


@pytest.mark.parametrize("H,Hkv,D,page", [(32, 8, 128, 16), (6, 2, 64, 8), (20, 1, 48, 16), (3, 3, 256, 32),
                                           (16, 4, 128, 64)])
@pytest.mark.parametrize("window", [0, 100])
@pytest.mark.parametrize("source", ["tensor", "partials"])
@pytest.mark.parametrize("lengths", ["mixed", "long"])
def test_decode_attention_from_the_projection(H, Hkv, D, page, window, source, lengths):
    """Decode steps hand the fused q/k/v projection to the attention kernel, which applies the
    per-head norm and the rotary encoding and writes the newest key and value itself: the same
    outputs and the same cache as the norm/rotary kernel followed by the attention kernel."""
    from tinyserve_b200.parts.rotary import Rotary
    o = ops()
    # "long": two requests with so many keys that there are more key ranges than a cluster takes
    kv_lens_of = {"mixed": [1, 64, 65, 300, 129, 700, 17, 128], "long": [3000, 2177]}
    if lengths == "long" and source == "tensor":
        pytest.skip("one pass over the long contexts is enough")
    kv_lens = kv_lens_of[lengths]
    B, width = len(kv_lens), (H + 2 * Hkv) * D
    K = 256
    x, w = rnd(B, K, seed=1, dtype=torch.bfloat16), rnd(width, K, seed=2, dtype=torch.bfloat16, scale=0.2)
    if source == "partials" and width >= 256:
        qkv = o._linear_tcgen05(x, w, False, splits=2, partials_only=True)
    else:
        qkv = o.linear(x, w)
    k = [rnd(n, Hkv, D, seed=10 + i, dtype=torch.bfloat16).cpu() for i, n in enumerate(kv_lens)]
    v = [rnd(n, Hkv, D, seed=30 + i, dtype=torch.bfloat16).cpu() for i, n in enumerate(kv_lens)]
    kc, vc, table = _paged(k, v, page, sum(-(-n // page) for n in kv_lens) + 3, seed=4)
    pos = torch.tensor([n - 1 for n in kv_lens], dtype=torch.int32).cuda()
    slots = torch.stack([table[b, (n - 1) // page] * page + (n - 1) % page for b, n in enumerate(kv_lens)]).int().cuda()
    dropped = 6 if B > 6 else 1
    slots[dropped] = -1                # this request writes nothing (its newest key is still used)
    rot = Rotary(D, 1e4, "half")
    rot.cos, rot.sin = (t.cuda() for t in Rotary.tables(D, 1e4, 4096))
    qw, kw = rnd(D, seed=5, dtype=torch.float32) + 1, rnd(D, seed=6, dtype=torch.float32) + 1
    cu = torch.arange(B + 1, dtype=torch.int32).cuda()
    ctx = SimpleNamespace(cu_q=cu, kv_lens=torch.tensor(kv_lens, dtype=torch.int32).cuda(), num_requests=B,
                          max_q_len=1, max_kv_len=max(kv_lens))
    view = SimpleNamespace(block_table=table, page_size=page, slot_mapping=slots)
    results = []
    for fused in (True, False):
        kc_i, vc_i = kc.clone(), vc.clone()
        launches = o.launch_count()
        out = o.attention_from_qkv(qkv, pos, H, Hkv, D, rot, qw, kw, 1e-6, kc_i, vc_i, view, ctx, D ** -0.5, window,
                                   fused=fused)
        results.append((out, kc_i, vc_i, o.launch_count() - launches))
    (out_f, kc_f, vc_f, n_f), (out_u, kc_u, vc_u, n_u) = results
    assert n_f < n_u, "fewer kernels"
    live = [b for b in range(B) if b != dropped]
    assert torch.equal(kc_f, kc_u) and torch.equal(vc_f, vc_u), "the same cache, bit by bit"
    assert (out_f[live].float() - out_u[live].float()).abs().max().item() <= 2.0 ** -7 * out_u.float().abs().max().item()
    # and both against the plain formulas in float64: per-head norm, rotary, attention over the old
    # keys and the newest one (the request without a slot too: the fused kernel uses its own newest
    # key although it writes none)
    full = o.materialize(qkv).double().cpu().view(B, H + 2 * Hkv, D)
    qh, kh, vh = full[:, :H], full[:, H:H + Hkv], full[:, H + Hkv:]
    def norm_rope(x, w, at):
        x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w.double().cpu()
        c, s_ = rot.cos.cpu()[at].double()[:, None], rot.sin.cpu()[at].double()[:, None]
        x1, x2 = x.chunk(2, -1)
        return torch.cat([x1 * c - x2 * s_, x2 * c + x1 * s_], -1)
    at = pos.long().cpu()
    qn = norm_rope(qh, qw, at).to(torch.bfloat16).double()
    kn, vn = norm_rope(kh, kw, at).to(torch.bfloat16), vh.to(torch.bfloat16)
    k_all = [torch.cat([k[b][:n - 1], kn[b][None]]) for b, n in enumerate(kv_lens)]
    v_all = [torch.cat([v[b][:n - 1], vn[b][None]]) for b, n in enumerate(kv_lens)]
    want = _attention_ref(qn, k_all, v_all, [1] * B, D ** -0.5, window)
    close(out_f, want, torch.bfloat16, "fused path against float64")
    close(out_u[live], want[live], torch.bfloat16, "two-kernel path against float64")


@pytest.mark.parametrize("D,H,Hkv", [(128, 8, 2), (64, 6, 1)])
@pytest.mark.parametrize("window", [0, 700])
def test_prefill_attention_long_prompt(D, H, Hkv, window):
    """A prompt of 2,500 tokens after a prefix of 300 (20 and more key tiles per block, uneven last
    query block), beside a short request; the reference runs on the GPU in 32-bit."""
    page = 16
    kv_lens, q_lens = [2800, 75], [2500, 75]
    k = [rnd(n, Hkv, D, seed=70 + i, dtype=torch.bfloat16).cpu() for i, n in enumerate(kv_lens)]
    v = [rnd(n, Hkv, D, seed=80 + i, dtype=torch.bfloat16).cpu() for i, n in enumerate(kv_lens)]
    q = rnd(sum(q_lens), H, D, seed=33, dtype=torch.bfloat16)
    kc, vc, table = _paged(k, v, page, sum(-(-n // page) for n in kv_lens) + 4, seed=6)
    want, at = [], 0
    for kb, vb, n in zip(k, v, q_lens):
        S = kb.shape[0]
        qq = q[at:at + n].float()                                       # [n, H, D]
        kk = kb.cuda().float().repeat_interleave(H // Hkv, 1)             # [S, H, D]
        vv = vb.cuda().float().repeat_interleave(H // Hkv, 1)
        sc = torch.einsum("thd,shd->hts", qq, kk) * D ** -0.5
        pos = torch.arange(S - n, S, device="cuda")[:, None]
        j = torch.arange(S, device="cuda")[None]
        vis = (j <= pos) & ((j > pos - window) if window else True)
        want.append(torch.einsum("hts,shd->thd", sc.masked_fill(~vis[None], float("-inf")).softmax(-1), vv))
        at += n
    for backend in ("tcgen05", "mma"):
        out = _run_attention(q, kc, vc, table, q_lens, kv_lens, page, D ** -0.5, window, None, backend)
        close(out, torch.cat(want), torch.bfloat16, f"long prompt ({backend})")
    assert ops().attention_tcgen05_error(D) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [1, 5])
@pytest.mark.parametrize("backend", ["mma", "simt"])
def test_attention_finds_one_far_key(dtype, splits, backend):
    """Among 700 keys one, on a page of its own early in the sequence, matches the query: the
    output must be that key's value."""
    H, Hkv, D, page, n, far = 4, 2, 32, 16, 700, 37
    k = rnd(n, Hkv, D, seed=1, dtype=dtype, scale=0.1).cpu()
    v = rnd(n, Hkv, D, seed=2, dtype=dtype).cpu()
    q = rnd(1, H, D, seed=3, dtype=dtype, scale=0.1)
    direction = torch.ones(D) / math.sqrt(D)
    k[far] = (direction * 40).to(dtype)
    q[0, :] = (direction * 40).to(dtype).cuda()
    if dtype == torch.float32 and backend == "mma":
        pytest.skip("float32 has one kernel")
    kc, vc, table = _paged([k], [v], page, 60, seed=2)
    run = lambda *a: _run_attention(*a, backend=backend)
    out = run(q, kc, vc, table, [1], [n], page, 1.0, 0, splits)
    want = v[far].repeat_interleave(H // Hkv, 0)
    assert (out[0].float().cpu() - want.float()).abs().max().item() < 1e-3
    # with a window that ends one key after it, it is hidden; one wider, it is seen
    hidden = run(q, kc, vc, table, [1], [n], page, 1.0, n - 1 - far, splits)
    assert (hidden[0].float().cpu() - want.float()).abs().max().item() > 0.1
    seen = run(q, kc, vc, table, [1], [n], page, 1.0, n - far, splits)
    assert (seen[0].float().cpu() - want.float()).abs().max().item() < 1e-3


def test_attention_refuses_what_it_cannot_do():
    o = ops()
    with pytest.raises(ValueError, match="head size"):
        o._attention(24)
    q = rnd(1, 3, 16)
    kc = torch.zeros(2, 2, 4, 16).cuda()
    view = SimpleNamespace(block_table=torch.zeros(1, 2, dtype=torch.int32).cuda(), page_size=4)
    ctx = SimpleNamespace(cu_q=torch.tensor([0, 1], dtype=torch.int32).cuda(),
                          kv_lens=torch.tensor([1], dtype=torch.int32).cuda(), num_requests=1,
                          max_q_len=1, max_kv_len=1)
    with pytest.raises(RuntimeError, match="heads"):
        o.paged_attention(q, kc, kc, view, ctx, 1.0)          # 3 heads over 2 KV heads
    with pytest.raises(RuntimeError, match="CUDA"):
        o.rmsnorm(torch.zeros(2, 8), torch.ones(8), 1e-6)


# ----------------------------------------------------------------------------- sampling
def test_sampler_greedy_and_ties():
    logits = rnd(5, 301, seed=1)
    logits[2, 17] = logits[2, 250] = 9.0          # a tie goes to the lowest id
    z = torch.zeros(5, device="cuda")
    out = ops().sample(logits, z, z.long(), z.int(), 0)
    want = logits.argmax(-1)
    assert out.tolist()[:2] == want.tolist()[:2] and out[2].item() == 17


def test_sampler_matches_the_documented_noise():
    import numpy as np
    import plain_qwen3 as plain
    B, V, seed = 6, 301, 99
    logits = rnd(B, V, seed=2, scale=2.0)
    temps = torch.tensor([0.8, 1.0, 0.3, 1.7, 0.0, 0.8]).cuda()
    streams = torch.tensor([5, 5, 2 ** 40 + 3, 9, 9, 123456789012], dtype=torch.int64).cuda()
    steps = torch.tensor([0, 1, 7, 3, 3, 0], dtype=torch.int32).cuda()
    out = ops().sample(logits, temps, streams, steps, seed).tolist()
    for i in range(B):
        row = logits[i].cpu()
        if temps[i] == 0:
            assert out[i] == int(row.argmax())
            continue
        noisy = row.double().numpy() / float(temps[i]) + plain.gumbel_noise(seed, int(streams[i]), int(steps[i]), V)
        top = np.sort(noisy)[-2:]
        if top[1] - top[0] > 1e-4:
            assert out[i] == int(np.argmax(noisy)), i
    # the same row in another batch, at another place, draws the same token
    again = ops().sample(logits[[3, 0]].contiguous(), temps[[3, 0]], streams[[3, 0]], steps[[3, 0]], seed)
    assert again.tolist() == [out[3], out[0]]


def test_sampler_top_k_top_p_keep_the_right_tokens():
    import plain_qwen3 as plain
    B, V = 8, 301
    logits = rnd(B, V, seed=3, scale=2.5)
    temps = torch.full((B,), 0.9).cuda()
    top_k = torch.tensor([1, 5, 0, 40, 0, 3, 300, 0], dtype=torch.int32).cuda()
    top_p = torch.tensor([1.0, 1.0, 0.5, 0.9, 0.05, 0.6, 0.99, 1.0]).cuda()
    kept = [plain.top_k_top_p_mask(logits[i].cpu(), 0.9, int(top_k[i]), float(top_p[i])) for i in range(B)]
    seen = [set() for _ in range(B)]
    for trial in range(200):
        steps = torch.full((B,), trial, dtype=torch.int32).cuda()
        out = ops().sample(logits, temps, torch.arange(B).cuda(), steps, 1, top_k=top_k, top_p=top_p)
        for i, t in enumerate(out.tolist()):
            seen[i].add(t)
            assert not torch.isinf(kept[i][t]), f"row {i} drew token {t}, which top-k/top-p drops"
    assert seen[0] == {int(logits[0].argmax())} and len(seen[4]) <= 2
    sizes = [int((~torch.isinf(k)).sum()) for k in kept]
    assert sizes[1] == 5 and len(seen[1]) >= 3 and len(seen[7]) > 10


def test_repetition_penalty():
    logits = torch.tensor([[2.0, -1.0, 0.5, 0.0], [1.0, 1.0, -1.0, -2.0], [3.0, 3.0, 3.0, 3.0]]).cuda()
    rows = torch.tensor([0, 2], dtype=torch.int32).cuda()
    ids = torch.tensor([[0, 1, -1], [3, -1, -1]], dtype=torch.int32).cuda()
    ops().apply_repetition_penalty(logits, rows, ids, torch.tensor([1.1, 2.0]).cuda())
    want = torch.tensor([[2.0 / 1.1, -1.1, 0.5, 0.0], [1.0, 1.0, -1.0, -2.0], [3.0, 3.0, 3.0, 1.5]])
    assert torch.allclose(logits.cpu(), want)


# ----------------------------------------------------------------------------- tcgen05 product
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 256, 256), (16, 384, 4096), (5, 200, 72), (17, 130, 136),
                                   (33, 4096, 1024), (64, 1000, 520), (100, 640, 192), (128, 128, 64),
                                   (8, 40000, 512), (3, 24576, 4096)])
@pytest.mark.parametrize("splits", [1, 2, 5])
@pytest.mark.parametrize("f32_out", [False, True])
@pytest.mark.parametrize("with_bias", [False, True])
def test_gemm_tcgen05(M, N, K, splits, f32_out, with_bias):
    o = ops()
    x, w = rnd(M, K, seed=1, dtype=torch.bfloat16), rnd(N, K, seed=2, dtype=torch.bfloat16, scale=0.1)
    splits = min(splits, -(-K // 64))
    bias = rnd(N, seed=3, dtype=torch.bfloat16 if M % 2 else torch.float32, scale=3.0) if with_bias else None
    out = o._linear_tcgen05(x, w, f32_out, splits=splits, bias=bias)
    torch.cuda.synchronize()
    assert o.gemm_tcgen05_error() == 0, "a block gave up on a wait"
    want = x.double() @ w.double().T + (bias.double() if with_bias else 0)
    close(out, want, torch.float32 if f32_out else torch.bfloat16, "tcgen05 gemm")
    again = o._linear_tcgen05(x, w, f32_out, splits=splits, bias=bias)
    assert torch.equal(out, again), "the split-K sum is the same every run"
    assert int(o._tile_counters(x.device).abs().sum()) == 0, "tile counters returned to zero"


def test_linear_picks_tcgen05_and_falls_back():
    o = ops()
    x, w = rnd(8, 4096, seed=1, dtype=torch.bfloat16), rnd(4096, 4096, seed=2, dtype=torch.bfloat16, scale=0.05)
    close(o.linear(x, w), x.double() @ w.double().T, torch.bfloat16, "decode-shaped")
    x2, w2 = rnd(8, 100, seed=3, dtype=torch.bfloat16), rnd(50, 100, seed=4, dtype=torch.bfloat16)
    close(o.linear(x2, w2), x2.double() @ w2.double().T, torch.bfloat16, "K not a multiple of 8: library")
    assert o.TCGEN05_MAX_TOKENS < 300
    x3 = rnd(300, 256, seed=5, dtype=torch.bfloat16)
    close(o.linear(x3, w[:64, :256].contiguous()), x3.double() @ w[:64, :256].double().T, torch.bfloat16, "many rows")
    # with a bias: the tcgen05 epilogue for few rows, the library's bias epilogue for many
    b = rnd(4096, seed=6, dtype=torch.bfloat16, scale=2.0)
    close(o.linear(x, w, b), x.double() @ w.double().T + b.double(), torch.bfloat16, "bias, few rows")
    x4 = rnd(300, 4096, seed=7, dtype=torch.bfloat16)
    close(o.linear(x4, w, b), x4.double() @ w.double().T + b.double(), torch.bfloat16, "bias, many rows")
    assert o.gemm_tcgen05_error() == 0


@pytest.mark.parametrize("M,N,K", [(8, 4096, 4096), (1, 256, 512), (13, 328, 1024), (16, 1024, 12288), (5, 136, 72)])
@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float32])
def test_product_with_residual_add_and_scaled_rows(M, N, K, wdtype):
    """The residual form of the tcgen05 product (its K cuts are a cluster that adds the partial
    sums, adds the residual and leaves rows without their norm factor) and the product that reads
    such rows and scales its result: together they are product + residual add + RMSNorm + product."""
    o = ops()
    x, w = rnd(M, K, seed=1, dtype=torch.bfloat16), rnd(N, K, seed=2, dtype=torch.bfloat16, scale=0.1)
    res = rnd(M, N, seed=3, scale=2.0)
    wn = rnd(N, seed=4, dtype=wdtype) + 1
    eps = 1e-5
    pending = o.linear(x, w, allow_pending=True)
    assert isinstance(pending, o.PendingProduct) and pending.shape == (M, N)
    close(pending.materialize(), x.double() @ w.double().T, torch.bfloat16, "materialize")
    r1 = res.clone()
    rows = o.add_rmsnorm(pending, r1, wn, eps, torch.bfloat16, scaled_ok=True)
    assert isinstance(rows, o.ScaledRows) and rows.shape == (M, N)
    v = res.double().cpu() + x.double().cpu() @ w.double().cpu().T
    assert (r1.double().cpu() - v).abs().max().item() < 1e-5 * max(1.0, v.abs().max().item()), "32-bit residual"
    want = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * wn.double().cpu()
    close(rows.materialize(), want, torch.bfloat16, "normalised rows")
    # without scaled_ok the same call gives the normalised rows themselves, by the ordinary kernels
    r2 = res.clone()
    plain = o.add_rmsnorm(o.linear(x, w, allow_pending=True), r2, wn, eps, torch.bfloat16)
    assert isinstance(plain, torch.Tensor)
    close(plain, want, torch.bfloat16, "unfused")
    # (a product that was not cut along K arrives rounded to bfloat16 on this path)
    assert (r2 - r1).abs().max().item() <= 2.0 ** -8 * (v - res.double().cpu()).abs().max().item()
    # the next product reads the rows without their factor and scales its result
    for N2, partials in ((384, False), (1152, True)):
        w2 = rnd(N2, N, seed=7, dtype=torch.bfloat16, scale=0.1)
        ref = rows.materialize().double().cpu() @ w2.double().cpu().T
        got = o.linear(rows, w2, allow_partials=partials)
        close(o.materialize(got), ref, torch.bfloat16, "scaled product")
        if wdtype == torch.float32:
            out32 = o.linear(rows, w2, out_float32=True)
            assert out32.dtype == torch.float32
            close(out32, ref, torch.bfloat16, "scaled product, 32-bit out")
    assert o.gemm_tcgen05_error() == 0


# ----------------------------------------------------------------------------- paired tcgen05 product
# (sizes: one tile and less; ragged edges in M, N and K; many tiles with a last wave that is cut
# along K for 74, 5 and 3 pairs; a K of one slice)
PAIR_SHAPES = [(65, 136, 72), (128, 256, 64), (130, 264, 520), (256, 512, 4096), (300, 1000, 136),
               (700, 2048, 1024), (1000, 4096, 512), (2048, 1536, 256)]


@pytest.mark.parametrize("M,N,K", PAIR_SHAPES)
@pytest.mark.parametrize("pairs", [74, 5, 3])
@pytest.mark.parametrize("halves", [1, 2])
@pytest.mark.parametrize("f32_out,with_bias", [(False, False), (True, True), (False, True)])
def test_gemm_pair(M, N, K, pairs, halves, f32_out, with_bias):
    o = ops()
    x, w = rnd(M, K, seed=1, dtype=torch.bfloat16), rnd(N, K, seed=2, dtype=torch.bfloat16, scale=0.1)
    bias = rnd(N, seed=3, dtype=torch.bfloat16 if M % 2 else torch.float32, scale=3.0) if with_bias else None
    out = o._linear_pair(x, w, f32_out, bias=bias, pairs=pairs, halves=halves)
    torch.cuda.synchronize()
    assert o.gemm_pair_error() == 0, "a block gave up on a wait"
    want = x.double() @ w.double().T + (bias.double() if with_bias else 0)
    close(out, want, torch.float32 if f32_out else torch.bfloat16, "paired gemm")
    # (the four issuing threads add into one accumulator in whatever order the tensor core takes
    # their instructions: two runs agree to the rounding of a 32-bit sum, not bit by bit)
    again = o._linear_pair(x, w, f32_out, bias=bias, pairs=pairs, halves=halves)
    close(again, want, torch.float32 if f32_out else torch.bfloat16, "paired gemm, second run")
    if f32_out:
        assert (again - out).abs().max().item() <= 1e-5 * want.abs().max().item()
    assert int(o._pair_scratch[str(x.device)][1].abs().sum()) == 0, "tile counters returned to zero"


@pytest.mark.parametrize("M,N,K,pairs", [(300, 1000, 12288, 7), (700, 1536, 16384, 20), (256, 2304, 20480, 74)])
@pytest.mark.parametrize("mode", ["plain", "gated", "residual"])
def test_gemm_pair_cuts_the_tiles_of_its_last_wave(M, N, K, pairs, mode):
    """With a long K the tiles of the last, partial wave are cut along K: the pairs add their
    parts to a sum in global memory (scratch, or the residual itself) and the block that arrives
    last finishes the tile.  The scratch and its counters are zero again afterwards."""
    import ctypes
    o = ops()
    if mode == "gated" and N % 128:
        pytest.skip("the gated form takes whole blocks of 64 gate and 64 up rows")
    lib = o._gemm_pair()
    lib.ts_gemm_pair_scratch.restype = ctypes.c_longlong
    need = lib.ts_gemm_pair_scratch(ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(pairs),
                                    ctypes.c_int(1), ctypes.c_int(0), None)
    assert need > 0, "this size is meant to cut tiles"
    x, w = rnd(M, K, seed=1, dtype=torch.bfloat16), rnd(N, K, seed=2, dtype=torch.bfloat16, scale=0.05)
    want = x.double() @ w.double().T
    if mode == "plain":
        out = o._linear_pair(x, w, pairs=pairs, halves=1)
    elif mode == "gated":
        out = o._linear_pair(x, w, gated=1, pairs=pairs, halves=1)
        full = want.view(M, N // 128, 2, 64)
        want = torch.nn.functional.silu(full[:, :, 0].reshape(M, N // 2)) * full[:, :, 1].reshape(M, N // 2)
    else:
        res, wn = rnd(M, N, seed=3, scale=2.0), rnd(N, seed=4) + 1
        r1 = res.clone()
        hprime, sumsq = o._linear_pair(x, w, residual=r1, norm_weight=wn, pairs=pairs, halves=1)
        v = res.double() + want
        # (a 32-bit sum over 12 to 20 thousand products: a few 1e-5 of the largest value)
        assert (r1.double() - v).abs().max().item() < 5e-5 * v.abs().max().item(), "32-bit residual"
        out = o.ScaledRows(hprime, sumsq, -(-N // 128), 1e-5).materialize()
        want = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5) * wn.double()
    torch.cuda.synchronize()
    assert o.gemm_pair_error() == 0
    close(out, want, torch.bfloat16, "paired gemm with cut tiles")
    scratch, counters = o._pair_scratch[str(x.device)]
    assert float(scratch.abs().max()) == 0.0 and int(counters.abs().sum()) == 0, "scratch and counters returned to zero"


@pytest.mark.parametrize("M,N,K", [(65, 128, 72), (200, 384, 520), (512, 1024, 1024), (1100, 6144, 256)])
@pytest.mark.parametrize("pairs", [74, 3])
@pytest.mark.parametrize("halves", [1, 2])
@pytest.mark.parametrize("activation", ["silu", "gelu_tanh"])
def test_gemm_pair_gated(M, N, K, pairs, halves, activation):
    """Weight rows alternate in blocks of 64 (gate, up); the epilogue applies act(gate) * up."""
    o = ops()
    x, w = rnd(M, K, seed=1, dtype=torch.bfloat16), rnd(N, K, seed=2, dtype=torch.bfloat16, scale=0.1)
    out = o._linear_pair(x, w, gated=o.ACTIVATIONS[activation] + 1, pairs=pairs, halves=halves)
    torch.cuda.synchronize()
    assert o.gemm_pair_error() == 0
    full = (x.double() @ w.double().T).view(M, N // 128, 2, 64)
    gate, up = full[:, :, 0].reshape(M, N // 2), full[:, :, 1].reshape(M, N // 2)
    act = torch.nn.functional.silu(gate) if activation == "silu" else torch.nn.functional.gelu(gate, approximate="tanh")
    close(out, act * up, torch.bfloat16, "gated paired gemm")


@pytest.mark.parametrize("M,N,K", [(65, 136, 72), (256, 4096, 1024), (300, 1000, 520), (1030, 2048, 256)])
@pytest.mark.parametrize("pairs,halves", [(74, 1), (74, 2), (3, 1), (3, 2), (74, 0)])
@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float32])
def test_gemm_pair_residual_and_scaled_rows(M, N, K, pairs, halves, wdtype):
    """The residual form (residual += x w^T in 32-bit, rows residual * norm weight and their sums
    of squares) and the forms that take such rows and scale their result by the norm factor."""
    o = ops()
    x, w = rnd(M, K, seed=1, dtype=torch.bfloat16), rnd(N, K, seed=2, dtype=torch.bfloat16, scale=0.1)
    res = rnd(M, N, seed=3, scale=2.0)
    wn = rnd(N, seed=4, dtype=wdtype) + 1
    eps = 1e-5
    r1 = res.clone()
    hprime, sumsq = o._linear_pair(x, w, residual=r1, norm_weight=wn, pairs=pairs, halves=halves)
    rows = o.ScaledRows(hprime, sumsq, -(-N // 128), eps)
    v = res.double().cpu() + x.double().cpu() @ w.double().cpu().T
    assert (r1.double().cpu() - v).abs().max().item() < 1e-5 * max(1.0, v.abs().max().item()), "32-bit residual"
    want = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * wn.double().cpu()
    close(rows.materialize(), want, torch.bfloat16, "normalised rows")
    normed = rows.materialize().double().cpu()
    w2 = rnd(384, N, seed=7, dtype=torch.bfloat16, scale=0.1)
    close(o._linear_pair(hprime, w2, scale=rows, pairs=pairs, halves=halves), normed @ w2.double().cpu().T, torch.bfloat16, "scaled product")
    full = (normed @ w2.double().cpu().T).view(M, 3, 2, 64)
    gated = torch.nn.functional.silu(full[:, :, 0].reshape(M, 192)) * full[:, :, 1].reshape(M, 192)
    close(o._linear_pair(hprime, w2, scale=rows, gated=1, pairs=pairs, halves=halves), gated, torch.bfloat16, "scaled gated product")
    assert o.gemm_pair_error() == 0


@pytest.mark.parametrize("M,N,K,splits", [(8, 4096, 1024, 4), (3, 328, 512, 2), (16, 6144, 512, 3), (40, 640, 256, 2)])
def test_split_partials_and_their_consumers(M, N, K, splits):
    """A product may stop at its split-K partial tiles; the next kernel adds them while it loads."""
    from tinyserve_b200.parts.rotary import Rotary
    o = ops()
    x, w = rnd(M, K, seed=1, dtype=torch.bfloat16), rnd(N, K, seed=2, dtype=torch.bfloat16, scale=0.1)
    want = x.double() @ w.double().T
    parts = o._linear_tcgen05(x, w, False, splits=splits, partials_only=True)
    assert isinstance(parts, o.SplitPartials) and parts.shape == (M, N)
    close(parts.materialize(), want, torch.bfloat16, "materialize")
    # residual add + norm straight from the partial tiles: the sum is never rounded to bfloat16
    res = rnd(M, N, seed=3, scale=2.0)
    wn = rnd(N, seed=4, dtype=torch.bfloat16) + 1
    r1 = res.clone()
    got = o.add_rmsnorm(parts, r1, wn, 1e-6, torch.bfloat16)
    v = res.double().cpu() + want.cpu()
    close(got, v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * wn.double().cpu(), torch.bfloat16, "norm")
    assert (r1.double().cpu() - v).abs().max().item() < 1e-3 * v.abs().max().item()
    rows = torch.tensor([M - 1, 0], dtype=torch.int32).cuda()
    r2 = res.clone()
    got2 = o.add_rmsnorm(parts, r2, wn, 1e-6, torch.bfloat16, rows=rows)
    assert torch.equal(got2, got[rows.long()]) and torch.equal(r2, res)
    # q/k norm + rotary + cache write straight from the partial tiles
    D = 64 if N % 64 == 0 else 8
    heads = N // D
    if heads >= 3 and heads % 3 == 0:
        H = Hkv = heads // 3
        rot = Rotary(D, 1e4, "half")
        rot.cos, rot.sin = (t.cuda() for t in Rotary.tables(D, 1e4, 64))
        pos = torch.arange(M, dtype=torch.int32).cuda()
        slots = torch.arange(16, 16 + M, dtype=torch.int32).cuda()
        qw, kw = rnd(D, seed=5, dtype=torch.bfloat16) + 1, rnd(D, seed=6, dtype=torch.bfloat16) + 1
        caches = [torch.zeros(8, Hkv, 16, D, dtype=torch.bfloat16).cuda() for _ in range(4)]
        q_a = o.qk_norm_rope_kvwrite(parts, pos, H, Hkv, D, rotary=rot, q_weight=qw, k_weight=kw, eps=1e-6,
                                     k_cache=caches[0], v_cache=caches[1], slot_mapping=slots, page_size=16)
        q_b = o.qk_norm_rope_kvwrite(parts.materialize(), pos, H, Hkv, D, rotary=rot, q_weight=qw, k_weight=kw,
                                     eps=1e-6, k_cache=caches[2], v_cache=caches[3], slot_mapping=slots, page_size=16)
        for a, b in ((q_a, q_b), (caches[0], caches[2]), (caches[1], caches[3])):
            assert (a.float() - b.float()).abs().max().item() <= 2e-2 * b.float().abs().max().item()
    assert o.gemm_tcgen05_error() == 0


# ----------------------------------------------------------------------------- index check
def test_index_check_neutralises_bad_indices_and_reports_them():
    """The device half of the debug pass: indices outside their buffers are replaced by harmless
    ones before any kernel uses them, and the status words say what was found.  (Nothing here
    reads or writes out of bounds: the check kernel only compares and rewrites the indices.)"""
    o = ops()
    dev = "cuda"
    i32 = lambda *v: torch.tensor(v, dtype=torch.int32, device=dev)
    words = o.status_words()
    assert not words.any()

    def step(**over):
        base = dict(token_ids=i32(5, 1, 2, -2), positions=i32(0, 1, 2, 7), logit_rows=i32(2, 3), cu_q=i32(0, 3, 4),
                    kv_lens=i32(3, 8), state_slots=i32(0, 1), slot_tokens=i32(4, 6, 0), num_tokens=4, num_requests=2,
                    num_logit_rows=2)
        base.update(over)
        view = SimpleNamespace(slot_mapping=over.get("slot_mapping", i32(16, 17, 18, 39)), page_size=8, max_blocks=2,
                               block_table=over.get("block_table", i32(2, 0, 4, 3).view(2, 2)), num_pages=5)
        return SimpleNamespace(groups=[view], **{k: v for k, v in base.items() if k not in ("slot_mapping", "block_table")})

    try:
        good = step()
        before = {k: v.clone() for k, v in vars(good).items() if isinstance(v, torch.Tensor)}
        o.sanitize_step(good, vocab_size=10, num_positions=16, max_kv_len=16, num_state_slots=2)
        torch.cuda.synchronize()
        assert not words.any(), "a step whose indices are fine is left alone"
        assert all(torch.equal(v, getattr(good, k)) for k, v in before.items())
        cases = [
            (dict(token_ids=i32(5, 10, 2, -2)), 1, lambda c: c.token_ids.tolist() == [5, 0, 2, -2]),
            (dict(token_ids=i32(5, 1, 2, -4)), 6, lambda c: c.token_ids.tolist() == [5, 1, 2, 0]),
            (dict(slot_tokens=i32(4, 60, 0)), 1, lambda c: c.slot_tokens.tolist() == [4, 0, 0]),
            (dict(positions=i32(0, 1, 16, 7)), 4, lambda c: c.positions.tolist() == [0, 1, 0, 7]),
            (dict(logit_rows=i32(2, 4)), 5, lambda c: c.logit_rows.tolist() == [2, 0]),
            (dict(state_slots=i32(0, 2)), 6, lambda c: c.state_slots.tolist() == [0, 0]),
            (dict(cu_q=i32(0, 5, 4)), 7, lambda c: c.cu_q.tolist() == [0, 0, 0] and c.kv_lens.tolist() == [0, 0]),
            (dict(kv_lens=i32(2, 8)), 7, lambda c: c.cu_q.tolist() == [0, 0, 0]),
            (dict(slot_mapping=i32(16, 17, 40, 39)), 2, lambda c: c.groups[0].slot_mapping.tolist() == [16, 17, -1, 39]),
            (dict(block_table=i32(2, 5, 4, -1).view(2, 2)), 3, lambda c: c.groups[0].block_table.tolist() == [[2, 0], [4, 0]]),
        ]
        for over, code, repaired in cases:
            ctx = step(**over)
            o.sanitize_step(ctx, vocab_size=10, num_positions=16, max_kv_len=16, num_state_slots=2)
            torch.cuda.synchronize()
            assert words[1] == code and words[0] == 0, (over, int(words[1]))
            assert repaired(ctx), over
            with pytest.raises(o.DeviceError):
                o.raise_on_device_error()
            words[:] = 0
    finally:
        words[:] = 0
