"""The allocation-free attention entry point, called through its exported C symbol.

Some callers of a kernel library cannot allocate device memory (a frozen memory pool, a
real-time loop, a plug-in that only gets its inputs and outputs).  For them
``ts_paged_attention_static_scratch`` keeps the split-KV scratch in a fixed array inside the
library.  This test calls it twice in a row with raw pointers and compares both results with
the ordinary entry point, which takes its scratch from the caller, and with the attention
formula evaluated in float64.  The file is named so that pytest collects it last."""
import ctypes
from ctypes import c_float, c_int, c_void_p
from types import SimpleNamespace

import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(seed, dtype, H, Hkv, D, page, kv_lens, q_lens):
    g = torch.Generator().manual_seed(seed)
    pages = sum(-(-n // page) for n in kv_lens) + 1
    kc = torch.randn(pages, Hkv, page, D, generator=g).to(dtype).cuda()
    vc = torch.randn(pages, Hkv, page, D, generator=g).to(dtype).cuda()
    max_blocks = max(-(-n // page) for n in kv_lens)
    table = torch.zeros(len(kv_lens), max_blocks, dtype=torch.int32)
    order = (torch.randperm(pages - 1, generator=g) + 1).tolist()
    for b, n in enumerate(kv_lens):
        for i in range(-(-n // page)):
            table[b, i] = order.pop()
    q = torch.randn(sum(q_lens), H, D, generator=g).to(dtype).cuda()
    cu = torch.tensor([0] + torch.tensor(q_lens).cumsum(0).tolist(), dtype=torch.int32).cuda()
    kv = torch.tensor(kv_lens, dtype=torch.int32).cuda()
    return q, kc, vc, table.cuda(), cu, kv


def _float64_attention(q, kc, vc, table, q_lens, kv_lens, page, scale):
    """softmax(q k^T * scale) v per request over its pages, causal from the end, in float64."""
    out, at = [], 0
    G = q.shape[1] // kc.shape[1]
    for b, (n, kv) in enumerate(zip(q_lens, kv_lens)):
        pages = table[b, :-(-kv // page)].long()
        k = kc[pages].double().permute(0, 2, 1, 3).reshape(-1, kc.shape[1], kc.shape[3])[:kv].repeat_interleave(G, 1)
        v = vc[pages].double().permute(0, 2, 1, 3).reshape(-1, vc.shape[1], vc.shape[3])[:kv].repeat_interleave(G, 1)
        s = torch.einsum("thd,shd->hts", q[at:at + n].double(), k) * scale
        pos = torch.arange(kv - n, kv, device=q.device)
        s = s.masked_fill(torch.arange(kv, device=q.device)[None] > pos[:, None], float("-inf"))
        out.append(torch.einsum("hts,shd->thd", s.softmax(-1), v))
        at += n
    return torch.cat(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_point_matches_the_ordinary_one(dtype):
    from tinyserve_b200.kernels import build, ops
    H, Hkv, D, page, splits = 8, 2, 64, 16, 4
    path = build.compile_unit("attention_simt.cu", {"TS_HEAD_DIM": D})
    lib = ctypes.CDLL(path)
    fn = lib.ts_paged_attention_static_scratch
    fn.restype = c_int
    lib.ts_last_error.restype = ctypes.c_char_p
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for call, (kv_lens, q_lens) in enumerate([([300, 77, 513], [1, 1, 1]), ([150, 40], [9, 40])]):
        q, kc, vc, table, cu, kv = _problem(call, dtype, H, Hkv, D, page, kv_lens, q_lens)
        ctx = SimpleNamespace(cu_q=cu, kv_lens=kv, num_requests=len(q_lens), max_q_len=max(q_lens),
                              max_kv_len=max(kv_lens))
        view = SimpleNamespace(block_table=table, page_size=page)
        want = ops.paged_attention(q, kc, vc, view, ctx, D ** -0.5, 0, num_splits=splits)
        out = torch.full_like(q, float("nan"))
        allocated = torch.cuda.memory_allocated()
        rc = fn(c_int(0 if dtype == torch.float32 else 1), c_void_p(q.data_ptr()), c_void_p(out.data_ptr()),
                c_void_p(kc.data_ptr()), c_void_p(vc.data_ptr()), c_void_p(table.data_ptr()),
                c_void_p(cu.data_ptr()), c_void_p(kv.data_ptr()), c_int(q.shape[0]), c_int(len(q_lens)),
                c_int(max(q_lens)), c_int(H), c_int(Hkv), c_int(page), c_int(table.stride(0)),
                c_float(D ** -0.5), c_int(0), c_int(splits), stream)
        assert rc == 0, lib.ts_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == allocated
        err = (out.float() - want.float()).abs().max().item()
        assert err <= tol * want.float().abs().max().item(), (call, err)
        exact = _float64_attention(q, kc, vc, table, q_lens, kv_lens, page, D ** -0.5)
        err = (out.double() - exact).abs().max().item()
        assert err <= tol * exact.abs().max().item(), ("against float64", call, err)
    # a call that needs more scratch than the array holds is refused, with the reason
    rc = fn(c_int(1), c_void_p(q.data_ptr()), c_void_p(out.data_ptr()), c_void_p(kc.data_ptr()),
            c_void_p(vc.data_ptr()), c_void_p(table.data_ptr()), c_void_p(cu.data_ptr()),
            c_void_p(kv.data_ptr()), c_int(4096), c_int(2), c_int(40), c_int(H), c_int(Hkv), c_int(page),
            c_int(table.stride(0)), c_float(1.0), c_int(0), c_int(8), stream)
    assert rc != 0 and b"static array holds" in lib.ts_last_error()
    # with one key range nothing is kept in the array, so no size is too large for it
    kv_lens, q_lens = [2100], [2100]
    q, kc, vc, table, cu, kv = _problem(9, dtype, H, Hkv, D, page, kv_lens, q_lens)
    assert q.shape[0] * H * (D + 2) > 2 ** 20
    out = torch.full_like(q, float("nan"))
    rc = fn(c_int(0 if dtype == torch.float32 else 1), c_void_p(q.data_ptr()), c_void_p(out.data_ptr()),
            c_void_p(kc.data_ptr()), c_void_p(vc.data_ptr()), c_void_p(table.data_ptr()), c_void_p(cu.data_ptr()),
            c_void_p(kv.data_ptr()), c_int(q.shape[0]), c_int(1), c_int(2100), c_int(H), c_int(Hkv), c_int(page),
            c_int(table.stride(0)), c_float(D ** -0.5), c_int(0), c_int(1), stream)
    assert rc == 0, lib.ts_last_error().decode()
    exact = _float64_attention(q, kc, vc, table, q_lens, kv_lens, page, D ** -0.5)
    assert (out.double() - exact).abs().max().item() <= tol * exact.abs().max().item()
