"""Python bindings of the CUDA kernels.  Every op here launches this package's own
sm_100a code through ctypes (matrix products of the bfloat16 path may go to cuBLAS, as
they do in tinyserve: serve.py:828-829).  There is no CPU path and no fallback: tensors
must live on a CUDA device and a missing compiler or library raises."""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

import torch

from . import build

ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}
SUPPORTED_HEAD_DIMS = tuple(range(16, 513, 16))
_DTYPE = {torch.float32: 0, torch.bfloat16: 1}

_launches = 0
#: bfloat16 matrix products of up to this many rows run on this package's TMA + tcgen05 kernel,
#: larger ones go to cuBLAS (measured on B200 at Qwen3-8B shapes, whole decode steps: 32 tokens
#: +8 %, 48 +4 %, 64 +2 % over cuBLAS)
TCGEN05_MAX_TOKENS = 64
#: bfloat16 attention is chosen by head size: the tcgen05 prefill kernel for these head sizes, the
#: mma.sync kernels (prefill of other head sizes, every decode) up to MMA_MAX_HEAD_DIM, the 32-bit
#: kernel above that
TCGEN05_HEAD_DIMS = (64, 128)
MMA_MAX_HEAD_DIM = 256
MMA_PREFILL_ROWS = 64           # query rows of a block of the mma prefill kernel (4 warps of 16)
#: the key ranges of a split-KV decode are the blocks of a thread-block cluster and merge through
#: distributed shared memory when there are at most this many; more are merged by a second kernel
#: (measured on B200 from CUDA graphs, 8 requests x 640 keys: 14.4 us with the second launch,
#: less in the cluster)
CLUSTER_MERGE_MAX_SPLITS = 8
#: the SM count all split heuristics were measured at; the device's own count is used at run time
MEASURED_NUM_SMS = 148
_num_sms = None


def num_sms() -> int:
    """Multiprocessors of the current device (148 where no device is visible)."""
    global _num_sms
    if _num_sms is None:
        if torch.cuda.is_available():
            _num_sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        else:
            return MEASURED_NUM_SMS
    return _num_sms


# ----------------------------------------------------------------------------- device status
# Kernels never trap: a bounded wait that ran out, or (in a bounds-checking build) an index outside
# its buffer, stores a code into a few words of pinned host memory; see common.cuh.
STATUS_WORDS = 8
_BOUNDS_CODES = {1: "a token id outside the vocabulary", 2: "a cache slot outside the pool",
                 3: "a page number outside the pool", 4: "a position outside the tables",
                 5: "a row outside the batch", 6: "a state slot outside the pool",
                 7: "a request index outside the batch"}
_status = None


def status_words():
    """The int32 status words (a numpy view): pinned host memory that every loaded library writes."""
    global _status
    if _status is None:
        t = torch.zeros(STATUS_WORDS, dtype=torch.int32)
        if torch.cuda.is_available():
            t = t.pin_memory()
        _status = (t, t.numpy())
    return _status[1]


def _register_status(lib):
    if hasattr(lib, "ts_set_status_words") and torch.cuda.is_available():
        status_words()
        if lib.ts_set_status_words(c_void_p(_status[0].data_ptr())) != 0:
            raise RuntimeError("a kernel library did not take the status words")


build.on_load.append(_register_status)


class DeviceError(RuntimeError):
    """A kernel reported that it gave up (a wait ran out) or met an index out of range."""


def raise_on_device_error() -> None:
    """Raise if any kernel has stored a status code since the process started.  Reads host memory
    only; call it after a synchronisation that covers the kernels in question.  The codes stay: an
    engine that has seen one does not go on."""
    w = status_words()
    if w[0]:
        raise DeviceError("a kernel gave up on a bounded wait (mbarrier): its results are not valid; "
                          "the engine stops")
    if w[1]:
        raise DeviceError(f"a kernel met {_BOUNDS_CODES.get(int(w[1]), 'an index out of range')}; "
                          "the access was skipped and the engine stops")


class SplitPartials:
    """The result of a matrix product as split-K partial tiles: the product's kernel stopped
    before adding them up, because the next kernel (residual add + norm, or the q/k norm + rotary
    kernel) adds them while it loads, which is cheaper than reducing inside the product.
    ``materialize()`` adds them up into an ordinary [M, N] tensor for any other consumer."""

    def __init__(self, data, splits, M, N, tile_t, dtype):
        self.data, self.splits, self.M, self.N, self.tile_t, self.dtype = data, splits, M, N, tile_t, dtype
        self.n_tiles, self.t_tiles = -(-N // 128), -(-M // tile_t)
        self.shape = (M, N)
        self.device = data.device

    def args(self):
        return (_ptr(self.data), c_int(self.splits), c_int(self.n_tiles), c_int(self.t_tiles),
                c_int(self.tile_t))

    def materialize(self):
        out = torch.empty(self.M, self.N, dtype=self.dtype, device=self.device)
        lib = _elementwise()
        _check(lib, lib.ts_reduce_partials(c_int(_DTYPE[self.dtype]), *self.args(), _ptr(out),
                                           c_int(self.M), c_int(self.N), _stream()))
        return out


_NO_PARTIALS = (c_void_p(0), c_int(0), c_int(0), c_int(0), c_int(0))

#: up to this many tokens the product before a residual add + norm does the add itself
#: (PendingProduct, ScaledRows), the gate/up product applies the activation in its epilogue and the
#: decode attention kernel takes the q/k/v projection as it is
FUSED_MAX_TOKENS = 16
FUSED_MAX_SPLITS = 8


class PendingProduct:
    """x @ weight^T that has not been launched yet.  ``linear(..., allow_pending=True)`` returns it
    for a few tokens, because the residual add + norm that usually follows can run in the
    product's own kernel: ``add_rmsnorm`` then launches the residual form of the tcgen05 kernel
    (the K cuts of a row tile are a thread-block cluster; they add their partial sums through
    distributed shared memory, add the residual and leave a ScaledRows).  For many tokens
    (``wide``) the paired kernel has the same form.  Any other consumer calls ``partials()`` or
    ``materialize()`` and gets the ordinary product."""

    def __init__(self, x, weight, wide=False):
        self.x, self.weight, self.wide = x, weight, wide         # wide: many tokens, the paired kernel
        self.shape = (x.shape[0], weight.shape[0])
        self.dtype, self.device = x.dtype, x.device

    def splits(self):
        M, K = self.x.shape
        return min(gemm_splits(M, self.weight.shape[0], K, partials=True), FUSED_MAX_SPLITS)

    def partials(self):
        if not self.wide and self.splits() > 1:
            return _linear_tcgen05(self.x, self.weight, False, partials_only=True)
        return self.materialize()

    def materialize(self):
        if self.wide:
            return _linear_pair(self.x, self.weight)
        return _linear_tcgen05(self.x, self.weight, False)


class ScaledRows:
    """Rows that still lack their RMSNorm factor: ``data`` [M, N] holds residual * norm_weight in
    bfloat16 and ``sumsq`` [tiles, 16] the sums of residual^2 over each 128 columns.  ``linear``
    takes it as x and scales every token's result by rsqrt(sum / N + eps) in its epilogue, which
    is the same product as with normalised rows; ``materialize()`` gives the normalised rows."""

    def __init__(self, data, sumsq, tiles, eps):
        self.data, self.sumsq, self.tiles, self.eps = data, sumsq, tiles, eps
        self.shape, self.dtype, self.device = tuple(data.shape), data.dtype, data.device

    @property
    def stride(self):
        """Tokens a tile's sums are apart: 16 from the product for few tokens, more from the paired one."""
        return self.sumsq.shape[1]

    def args(self):
        return (_ptr(self.sumsq), c_int(self.tiles), c_float(self.eps))

    def args_wide(self):
        return (_ptr(self.sumsq), c_int(self.tiles), c_int(self.stride), c_float(self.eps))

    def materialize(self):
        out = torch.empty_like(self.data)
        lib = _elementwise()
        _check(lib, lib.ts_scale_rows(_ptr(self.data), *self.args_wide(), _ptr(out), c_int(self.shape[0]),
                                      c_int(self.shape[1]), _stream()))
        return out


_NO_SCALE = (c_void_p(0), c_int(0), c_float(0.0))


def materialize(x):
    """An ordinary tensor from what a product or a norm returned."""
    return x.materialize() if isinstance(x, (SplitPartials, PendingProduct, ScaledRows)) else x


def launch_count() -> int:
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def require_device(device) -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("tinyserve_b200 runs on a CUDA device only (sm_100a); no GPU is visible "
                           "and there is no CPU path")
    if torch.device(device).type != "cuda":
        raise RuntimeError(f"tinyserve_b200 runs on CUDA devices only, got {device!r}")


_STREAM = None


def _stream():
    if _STREAM is not None:
        return _STREAM
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """Looks the current CUDA stream up once for all ops launched inside the scope (the lookup
    costs more than a kernel launch).  The current stream must not change inside the scope."""

    def __enter__(self):
        global _STREAM
        self._outer = _STREAM
        _STREAM = c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _STREAM
        _STREAM = self._outer
        return False


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _check(lib, code, n=1):
    if code != 0:
        raise RuntimeError(lib.ts_last_error().decode())
    count_launches(n)


def _dt(t):
    try:
        return _DTYPE[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; kernels take float32 and bfloat16") from None


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("kernel operands must be CUDA tensors: there is no CPU path")


def _vec_flag(w, like):
    """Norm weights are float32 or of the activations' dtype."""
    if w.dtype == torch.float32:
        return 1
    if w.dtype == torch.bfloat16:
        return 0
    raise TypeError(f"norm weight dtype {w.dtype} is not supported")


# ----------------------------------------------------------------------------- libraries
def _elementwise():
    return build.load_unit("elementwise.cu")


def _gemm():
    return build.load_unit("gemm_simt.cu")


def _gemm_tcgen05():
    return build.load_unit("gemm_tcgen05.cu")


_counters: dict = {}


def _tile_counters(device):
    """Zeroed tile counters of the split-K reduction; the kernel returns them to zero."""
    key = str(device)
    if key not in _counters:
        _counters[key] = torch.zeros(16384, dtype=torch.int32, device=device)
    return _counters[key]


def gemm_splits(M, N, K, partials=False):
    """Cuts along K of the tiled product, so that a product with few 128-row tiles still fills
    the SMs.  When the product reduces its own partial tiles: about 160 blocks, at least four
    64-wide slices per cut, wide token tiles cut at most in two (their partial tiles are large).
    When it hands the partial tiles on (``partials``): all 2 x 148 block slots, at most 8 cuts
    (measured on B200 at 8 tokens: 6144x4096 best at 6, 4096x4096 and 4096x12288 at 8)."""
    tile_t = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
    tiles = -(-N // 128) * -(-M // tile_t)
    slices = -(-K // 64)
    if tiles >= num_sms():
        return 1
    if partials:
        splits = max(1, min(2 * num_sms() // tiles, slices // 4, 8))
    else:
        splits = max(1, min(-(-160 // tiles), slices // 4, 16))
        if tile_t >= 64:
            splits = min(splits, 2)
    per = -(-slices // splits)
    return -(-slices // per)           # no cut without a slice


def gemm_tcgen05_error() -> int:
    """1 if a block of the tcgen05 kernel ever gave up on a wait (synchronises)."""
    return _gemm_tcgen05().ts_gemm_tcgen05_error()


def _tcgen05_ok(x, weight):
    return (x.shape[0] <= TCGEN05_MAX_TOKENS and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and weight.stride(1) == 1 and x.stride(0) % 8 == 0
            and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)


#: From this many tokens on the gate/up product runs on the paired tcgen05 kernel with the
#: activation in its epilogue.  Measured inside a whole prefill of Qwen3-8B shapes, warm, against
#: the library product + activation kernel: 2,048 tokens +3 %, 4,096 tokens +4.5 %.  Only for
#: rows of PAIR_GATED_MIN_K elements and more: a tile's epilogue (9 to 14 us beside running MMAs)
#: hides behind a mainloop of 64 slices of K, not behind one of 16 (Qwen3-0.6B shapes: slower).
PAIR_GATED_MIN_TOKENS = 2048
PAIR_GATED_MAX_TOKENS = 6144     # (at 8,192 tokens the library's product is 11 % faster, which is what the activation kernel costs)
PAIR_GATED_MIN_K = 4096
#: From this many tokens on every product of a layer runs on the paired kernel, with the residual
#: add, the norm factor and the activation in the products' epilogues.  Off: inside a whole
#: prefill the other three products are 2 to 8 % slower than the library's with the kernels
#: between them (their tiles do not fill whole waves of SM pairs); tests turn it on.
PAIR_MIN_TOKENS = 10 ** 9


def _pair_ok(x, weight):
    return (x.shape[1] % 8 == 0 and weight.shape[0] % 8 == 0 and x.stride(1) == 1 and weight.stride(1) == 1
            and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0)


def _tile_t(M):
    return 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128


def _linear_tcgen05(x, weight, out_float32, splits=None, partials_only=False, scale=None, gated=0, bias=None):
    """``scale``: the ScaledRows whose ``data`` is ``x``; ``gated``: activation code + 1 of the
    gated epilogue (out [M, N / 2]); ``bias`` [N]: added in the epilogue (not with the others)."""
    M, K = x.shape
    N = weight.shape[0]
    out_cols = N // 2 if gated else N
    out = None if partials_only else torch.empty(
        M, out_cols, dtype=torch.float32 if out_float32 else torch.bfloat16, device=x.device)
    lib = _gemm_tcgen05()
    lib.ts_gemm_tcgen05_scratch.restype = c_longlong
    if splits is None:
        splits = gemm_splits(M, N, K, partials=partials_only)
    if partials_only and splits < 2:
        raise ValueError("partial tiles need at least two splits")
    partials = counters = None
    if splits > 1:
        need = lib.ts_gemm_tcgen05_scratch(c_int(M), c_int(N), c_int(splits))
        partials = torch.empty(need, dtype=torch.float32, device=x.device)
        counters = None if partials_only else _tile_counters(x.device)
    if scale is not None or gated:
        if bias is not None:
            raise ValueError("the scaled-rows and gated products take no bias")
        _check(lib, lib.ts_gemm_tcgen05_fused(
            _ptr(x), _ptr(weight), _ptr(out), c_int(M), c_int(N), c_int(K), c_longlong(x.stride(0)),
            c_longlong(weight.stride(0)), c_longlong(out_cols), c_int(1 if out_float32 else 0), c_int(splits),
            _ptr(partials), _ptr(counters), *(scale.args() if scale is not None else _NO_SCALE), None, None,
            c_int(0), None, None, c_int(gated), _stream()))
    else:
        _check(lib, lib.ts_gemm_tcgen05(_ptr(x), _ptr(weight), _ptr(out), c_int(M), c_int(N), c_int(K),
                                        c_longlong(x.stride(0)), c_longlong(weight.stride(0)), c_longlong(N),
                                        c_int(1 if out_float32 else 0), c_int(splits), _ptr(partials),
                                        _ptr(counters), _ptr(bias),
                                        c_int(_vec_flag(bias, torch.bfloat16) if bias is not None else 0), _stream()))
    if partials_only:
        return SplitPartials(partials, splits, M, N, _tile_t(M), torch.bfloat16)
    return out


def _gemm_pair():
    return build.load_unit("gemm_pair_tcgen05.cu")


def gemm_pair_error() -> int:
    """1 if a block of the paired tcgen05 kernel ever gave up on a wait (synchronises)."""
    return _gemm_pair().ts_gemm_pair_error()


_pair_scratch: dict = {}
_pair_count: list = []


def gemm_pairs() -> int:
    """Pairs of blocks of the paired product that the device holds at once (74 on a B200 with all
    148 SMs in pairs)."""
    if not _pair_count:
        n = _gemm_pair().ts_gemm_pair_max_pairs()
        _pair_count.append(n if n > 0 else num_sms() // 2)
    return _pair_count[0]


def _pair_workspace(lib, M, N, K, pairs, halves, out_float32, device):
    """Where the parts of the cut tiles of the last wave are added up, and their counters: zero
    between products (the kernel leaves them so).  One buffer per device, grown on demand:
    products of one stream run one after the other."""
    counters = c_int(0)
    lib.ts_gemm_pair_scratch.restype = c_longlong
    need = lib.ts_gemm_pair_scratch(c_int(M), c_int(N), c_int(K), c_int(pairs), c_int(halves), c_int(1 if out_float32 else 0), ctypes.byref(counters))
    key = str(device)
    have = _pair_scratch.get(key)
    if have is None or have[0].numel() < need or have[1].numel() < counters.value:
        if torch.cuda.is_current_stream_capturing():
            # (a buffer made during a capture belongs to the graph's pool: it must not outlive it here)
            raise RuntimeError("the paired product's scratch would have to grow inside a graph capture: "
                               "run the shape once before it is captured")
        grow = max(need, have[0].numel() if have else 0, 1)
        have = (torch.zeros(grow, dtype=torch.float32, device=device),
                torch.zeros(max(counters.value, 1024), dtype=torch.int32, device=device))
        _pair_scratch[key] = have
    return have


def _linear_pair(x, weight, out_float32=False, bias=None, scale=None, gated=0, residual=None, norm_weight=None,
                 pairs=None, halves=0):
    """The product for many tokens on pairs of SMs (csrc/gemm_pair_tcgen05.cu).  Plain: returns
    out [M, N]; ``bias`` [N]; ``scale`` the ScaledRows whose ``data`` is ``x``.  ``gated``:
    activation code + 1, out [M, N / 2].  ``residual`` (float32 [M, N], in place) with
    ``norm_weight``: returns (hprime, sumsq) of the new residual.  ``halves``: tiles of 256 (1) or
    512 (2) weight rows, 0: the kernel's estimate decides."""
    M, K = x.shape
    N = weight.shape[0]
    lib = _gemm_pair()
    pairs = pairs or gemm_pairs()
    scratch, counters = _pair_workspace(lib, M, N, K, pairs, halves, out_float32, x.device)
    out = hprime = sumsq = None
    stride = -(-M // 4) * 4
    if residual is not None:
        hprime = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        sumsq = torch.empty(-(-N // 128), stride, dtype=torch.float32, device=x.device)
    else:
        out = torch.empty(M, N // 2 if gated else N, dtype=torch.float32 if out_float32 else torch.bfloat16,
                          device=x.device)
    _check(lib, lib.ts_gemm_pair(
        _ptr(x), _ptr(weight), _ptr(out), c_int(M), c_int(N), c_int(K), c_longlong(x.stride(0)),
        c_longlong(weight.stride(0)), c_longlong(out.stride(0) if out is not None else 0),
        c_int(1 if out_float32 else 0), _ptr(bias),
        c_int(_vec_flag(bias, torch.bfloat16) if bias is not None else 0),
        *(scale.args_wide() if scale is not None else (c_void_p(0), c_int(0), c_int(0), c_float(0.0))),
        c_int(gated), _ptr(residual), _ptr(norm_weight),
        c_int(_vec_flag(norm_weight, torch.bfloat16) if norm_weight is not None else 0), _ptr(hprime), _ptr(sumsq),
        c_int(stride), _ptr(scratch), c_longlong(scratch.numel()), _ptr(counters), c_int(counters.numel()),
        c_int(pairs), c_int(halves), _stream()))
    if residual is not None:
        return hprime, sumsq
    return out


def _attention(head_dim: int):
    if head_dim not in SUPPORTED_HEAD_DIMS:
        raise ValueError(f"head size {head_dim} is not supported: attention takes multiples of 16 "
                         f"up to {SUPPORTED_HEAD_DIMS[-1]}")
    return build.load_unit("attention_simt.cu", {"TS_HEAD_DIM": head_dim})


def _attention_mma(head_dim: int):
    return build.load_unit("attention_mma.cu", {"TS_HEAD_DIM": head_dim})


def _attention_tcgen05(head_dim: int):
    return build.load_unit("attention_tcgen05.cu", {"TS_HEAD_DIM": head_dim})


def attention_tcgen05_error(head_dim: int) -> int:
    """1 if a block of the tcgen05 attention kernel ever gave up on a wait (synchronises)."""
    return _attention_tcgen05(head_dim).ts_attention_tcgen05_error()


def attention_mma_error(head_dim: int) -> int:
    """1 if a block of the TMA decode kernel ever gave up on a wait (synchronises)."""
    return _attention_mma(head_dim).ts_attention_mma_error()


def _sampler():
    return build.load_unit("sampler.cu")


def units_for(head_dims) -> list:
    """The (source, defines) units a model with these head sizes needs."""
    units = [("elementwise.cu", {}), ("gemm_simt.cu", {}), ("gemm_tcgen05.cu", {}), ("gemm_pair_tcgen05.cu", {}),
             ("sampler.cu", {})]
    units += [("attention_simt.cu", {"TS_HEAD_DIM": d}) for d in sorted(set(head_dims))]
    units += [("attention_mma.cu", {"TS_HEAD_DIM": d}) for d in sorted(set(head_dims))
              if d <= MMA_MAX_HEAD_DIM]
    units += [("attention_tcgen05.cu", {"TS_HEAD_DIM": d}) for d in sorted(set(head_dims))
              if d in TCGEN05_HEAD_DIMS]
    return units


# ----------------------------------------------------------------------------- ops
def block_tables_step(resident, pairs, num_pairs, step_tables, state_slots, num_requests):
    """Apply a step's block-table changes to the resident rows and gather the rows of the step's
    requests.  resident int32 [G, slots + 1, max_blocks]; pairs int32 [capacity, 2] (flat index
    into resident, page); num_pairs int32 [1]; step_tables int32 [G, max_requests, max_blocks];
    state_slots int32 [>= num_requests]: all on the device.  Two small launches."""
    _cuda(resident, pairs, num_pairs, step_tables, state_slots)
    G, slots1, max_blocks = resident.shape
    lib = _elementwise()
    _check(lib, lib.ts_block_tables_step(
        _ptr(resident), _ptr(pairs), _ptr(num_pairs), c_int(pairs.shape[0]), _ptr(step_tables), _ptr(state_slots),
        c_int(num_requests), c_int(step_tables.shape[1]), c_int(slots1 - 1), c_int(max_blocks), c_int(G), _stream()), 2)


def sanitize_step(ctx, vocab_size, num_positions, max_kv_len, num_state_slots):
    """The device half of the index check (see csrc/elementwise.cu): every index of the step in
    ``ctx`` that lies outside its buffer is replaced by a harmless one and reported through the
    status words.  One small kernel, plus one per cache group."""
    lib = _elementwise()
    _cuda(ctx.token_ids, ctx.positions, ctx.cu_q, ctx.kv_lens, ctx.state_slots)
    _check(lib, lib.ts_sanitize_step(
        _ptr(ctx.token_ids), c_int(ctx.num_tokens), c_int(vocab_size), _ptr(ctx.slot_tokens),
        c_int(num_state_slots), _ptr(ctx.positions), c_int(num_positions), _ptr(ctx.logit_rows),
        c_int(ctx.num_logit_rows), _ptr(ctx.cu_q), _ptr(ctx.kv_lens), c_int(ctx.num_requests), c_int(max_kv_len),
        _ptr(ctx.state_slots), _stream()))
    for view in ctx.groups:
        _check(lib, lib.ts_sanitize_group(
            _ptr(view.slot_mapping), c_int(ctx.num_tokens), c_longlong(view.num_pages * view.page_size),
            _ptr(view.block_table), c_int(ctx.num_requests), c_int(view.max_blocks),
            c_int(view.block_table.stride(0)), c_int(view.num_pages), _stream()))


def embed_lookup(table, ids, slot_tokens=None):
    """float32 [T, n] = table[ids]; ids int32.  An id < 0 names a state slot (-1 - slot) whose
    last sampled token is read from ``slot_tokens`` on the device."""
    _cuda(table, ids, slot_tokens)
    T, n = ids.shape[0], table.shape[1]
    out = torch.empty(T, n, dtype=torch.float32, device=table.device)
    lib = _elementwise()
    _check(lib, lib.ts_embed_lookup(c_int(_dt(table)), _ptr(table), _ptr(ids), _ptr(out), c_int(T),
                                    c_int(n), c_int(table.shape[0]), _ptr(slot_tokens), _stream()))
    return out


def _product_add_residual(pending, residual, weight, eps):
    """The residual form of the tcgen05 product: residual += x w^T inside the product's kernel;
    returns the ScaledRows of the new residual for the norm with ``weight``."""
    x, w = pending.x, pending.weight
    M, K = x.shape
    N = w.shape[0]
    tiles = -(-N // 128)
    if pending.wide:
        hprime, sumsq = _linear_pair(x, w, residual=residual, norm_weight=weight)
        return ScaledRows(hprime, sumsq, tiles, eps)
    hprime = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    sumsq = torch.empty(tiles, 16, dtype=torch.float32, device=x.device)
    lib = _gemm_tcgen05()
    _check(lib, lib.ts_gemm_tcgen05_fused(
        _ptr(x), _ptr(w), None, c_int(M), c_int(N), c_int(K), c_longlong(x.stride(0)), c_longlong(w.stride(0)),
        c_longlong(N), c_int(0), c_int(pending.splits()), None, None, *_NO_SCALE, _ptr(residual), _ptr(weight),
        c_int(_vec_flag(weight, torch.bfloat16)), _ptr(hprime), _ptr(sumsq), c_int(0), _stream()))
    return ScaledRows(hprime, sumsq, tiles, eps)


def add_rmsnorm(x, residual, weight, eps, out_dtype, rows=None, scaled_ok=False):
    """residual (float32, in place) += x; returns rmsnorm(residual) * weight as ``out_dtype``.
    ``x`` None: no add; ``x`` may be the SplitPartials or the PendingProduct of a product.  With
    ``rows`` (int32) only those rows are normalised and returned, and the residual is left as it
    is.  With ``scaled_ok`` the caller takes a ScaledRows as well (it hands it to ``linear``)."""
    if isinstance(x, PendingProduct):
        if (scaled_ok and rows is None and out_dtype == torch.bfloat16 and x.shape == tuple(residual.shape)
                and residual.dtype == torch.float32 and residual.is_contiguous()):
            _cuda(residual, weight)
            return _product_add_residual(x, residual, weight, eps)
        x = x.partials()
    parts = _NO_PARTIALS
    if isinstance(x, SplitPartials):
        if x.shape != tuple(residual.shape):
            raise TypeError("add_rmsnorm: the partial tiles do not have the residual's shape")
        parts, x = x.args(), None
    _cuda(x, residual, weight, rows)
    if residual.dtype != torch.float32 or not residual.is_contiguous():
        raise TypeError("the residual stream is contiguous float32")
    if x is not None and (x.dtype != out_dtype or not x.is_contiguous() or x.shape != residual.shape):
        raise TypeError("add_rmsnorm: x must be contiguous, of the compute dtype and of the residual's shape")
    n = residual.shape[1]
    num_out = residual.shape[0] if rows is None else rows.shape[0]
    out = torch.empty(num_out, n, dtype=out_dtype, device=residual.device)
    lib = _elementwise()
    _check(lib, lib.ts_add_rmsnorm(c_int(_DTYPE[out_dtype]), _ptr(x), _ptr(residual), _ptr(weight),
                                   c_int(_vec_flag(weight, out_dtype)), c_float(eps), _ptr(out),
                                   _ptr(rows), c_int(num_out), c_int(n),
                                   c_int(0 if rows is not None else 1), *parts, _stream()))
    return out


def rmsnorm(x, weight, eps, out=None):
    _cuda(x, weight)
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    out = torch.empty_like(x2) if out is None else out
    lib = _elementwise()
    _check(lib, lib.ts_rmsnorm(c_int(_dt(x2)), _ptr(x2), _ptr(weight), c_int(_vec_flag(weight, x.dtype)),
                               c_float(eps), _ptr(out), c_int(x2.shape[0]), c_int(shape[-1]), _stream()))
    return out.view(shape)


def gated_activation(gate_up, activation="silu", block=0):
    """[rows, 2 I] -> act(gate) * up, [rows, I].  ``block`` 0: the input is gate | up; else gate
    and up columns alternate in blocks of ``block`` (see gated_linear)."""
    gate_up = materialize(gate_up)
    _cuda(gate_up)
    rows, two_i = gate_up.shape
    out = torch.empty(rows, two_i // 2, dtype=gate_up.dtype, device=gate_up.device)
    lib = _elementwise()
    _check(lib, lib.ts_gated_activation(c_int(_dt(gate_up)), _ptr(gate_up), _ptr(out), c_int(rows),
                                        c_int(two_i // 2), c_int(ACTIVATIONS[activation]), c_int(block), _stream()))
    return out


#: rows of gate and up alternate in blocks of this many in a fused gate/up weight: half a 128-row
#: tile of the tcgen05 product
GATED_BLOCK = 64


def gated_linear(x, weight, activation="silu", block=0):
    """act(gate) * up of x @ weight^T, [M, N / 2].  weight [N, K] holds gate rows then up rows
    (``block`` 0) or alternates them in blocks of ``block`` rows.  With blocks of GATED_BLOCK, up
    to FUSED_MAX_TOKENS tokens and a product that needs no cut along K, the tcgen05 product does
    the activation in its epilogue; otherwise the product is followed by the activation kernel.  x may be the
    ScaledRows that add_rmsnorm returned."""
    rows = x.data if isinstance(x, ScaledRows) else x
    N, K = weight.shape
    if (block == GATED_BLOCK and N % 128 == 0 and isinstance(rows, torch.Tensor)
            and rows.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and _pair_ok(rows, weight)
            and (rows.shape[0] >= PAIR_MIN_TOKENS
                 or (rows is x and PAIR_GATED_MIN_TOKENS <= rows.shape[0] <= PAIR_GATED_MAX_TOKENS
                     and K >= PAIR_GATED_MIN_K))):
        _cuda(rows, weight)
        return _linear_pair(rows, weight, gated=ACTIVATIONS[activation] + 1, scale=x if rows is not x else None)
    if (block == GATED_BLOCK and N % 128 == 0 and isinstance(rows, torch.Tensor)
            and rows.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and _tcgen05_ok(rows, weight)
            and rows.shape[0] <= FUSED_MAX_TOKENS          # measured: at 64 tokens the epilogue costs 9 % of the step
            and gemm_splits(rows.shape[0], N, K) == 1):
        _cuda(rows, weight)
        return _linear_tcgen05(rows, weight, False, splits=1, gated=ACTIVATIONS[activation] + 1,
                               scale=x if rows is not x else None)
    return gated_activation(linear(x, weight), activation, block)


def qk_norm_rope_kvwrite(qkv, positions, num_heads, num_kv_heads, head_dim, rotary=None,
                         q_weight=None, k_weight=None, eps=0.0, k_cache=None, v_cache=None,
                         slot_mapping=None, page_size=0):
    """Per-head norm of q and k, rotary encoding, q to a [T, H, D] tensor (returned), k and v
    to the cache slots of ``slot_mapping`` (None: nothing is written)."""
    parts, dtype = _NO_PARTIALS, qkv.dtype
    if isinstance(qkv, SplitPartials):
        if head_dim % 2:
            qkv = qkv.materialize()
        else:
            parts = qkv.args()
    T = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise ValueError("qkv must be [T, (H + 2 Hkv) * D]")
    device = qkv.device
    if parts is _NO_PARTIALS:
        if not qkv.is_contiguous():
            raise ValueError("qkv must be contiguous")
    else:
        qkv = None
    _cuda(qkv, positions, k_cache, v_cache, slot_mapping)
    q = torch.empty(T, num_heads, head_dim, dtype=dtype, device=device)
    cos = rotary.cos if rotary is not None else None
    sin = rotary.sin if rotary is not None else None
    rot = rotary.rotary_dim if rotary is not None else 0
    inter = int(rotary.interleaved) if rotary is not None else 0
    if k_cache is not None and k_cache.dtype != dtype:
        raise TypeError("cache and activations differ in dtype")
    flag = _vec_flag(q_weight, dtype) if q_weight is not None else 0
    if q_weight is not None and k_weight.dtype != q_weight.dtype:
        raise TypeError("q and k norm weights differ in dtype")
    lib = _elementwise()
    _check(lib, lib.ts_qk_norm_rope_kvwrite(
        c_int(_DTYPE[dtype]), _ptr(qkv), _ptr(q), _ptr(positions), _ptr(cos), _ptr(sin), c_int(rot),
        c_int(inter), _ptr(q_weight), _ptr(k_weight), c_int(flag), c_float(eps), c_int(T),
        c_int(num_heads), c_int(num_kv_heads), c_int(head_dim), _ptr(k_cache), _ptr(v_cache),
        _ptr(slot_mapping), c_int(page_size), *parts, _stream()))
    return q


def attention_splits(num_requests, max_q_len, max_kv_len, num_heads, num_kv_heads):
    """How many key ranges a launch is cut into so that a small batch still fills the SMs
    (tinykernels.py:865-889, for 148 SMs)."""
    group = num_heads // num_kv_heads
    per_tile = 32 // group if group < 32 else 1
    blocks = -(-max_q_len // per_tile) * num_kv_heads * -(-group // 32) * num_requests
    if blocks >= 2 * num_sms() or max_kv_len < 256:
        return 1
    want = -(-2 * num_sms() // blocks)
    return max(1, min(want, max_kv_len // 128, 32))


class AttentionWork:
    """The work lists of a step's attention launches, built once per step on the host."""
    __slots__ = ("tile_req", "tile_q0", "num_tiles", "dec_req", "dec_tok", "num_decode", "max_decode_kv")


def cut_attention_work(cu, kv, num_requests, queries_per_tile, split_decodes=True):
    """The host half: (tile_req, tile_q0, dec_req, dec_tok, longest decode context) as lists.
    Requests with several tokens are cut into blocks of ``queries_per_tile`` queries, (request,
    first query) each, heaviest (most keys) first, so that a long portion beside many short
    requests launches no block for nothing.  With ``split_decodes``, requests of one token are
    listed apart, (request, token) each, longest context first: they go to the decode kernel,
    which does not spend a block of rows on one query."""
    tiles, decodes = [], []
    for b in range(num_requests):
        n = cu[b + 1] - cu[b]
        if n == 1 and split_decodes:
            decodes.append((kv[b], b, cu[b]))
            continue
        for q0 in range(0, n, queries_per_tile):
            tiles.append((kv[b] - n + q0, b, q0))
    tiles.sort(reverse=True)
    decodes.sort(reverse=True)
    return ([t[1] for t in tiles], [t[2] for t in tiles], [d[1] for d in decodes], [d[2] for d in decodes],
            decodes[0][0] if decodes else 0)


def attention_work(ctx, queries_per_tile, device, split_decodes=True):
    """A step's attention work lists (int32 device tensors) for blocks of ``queries_per_tile``
    queries.  The engine's step function packs them with the rest of the step (one upload) for
    the tile sizes its mixers announce; for any other caller they are cut and uploaded here."""
    cache = getattr(ctx, "tile_cache", None)
    key = (queries_per_tile, split_decodes)
    if cache is not None and key in cache:
        return cache[key]
    host = getattr(ctx, "host", None) or {}
    cu = host.get("cu_q") or ctx.cu_q.tolist()
    kv = host.get("kv_lens") or ctx.kv_lens.tolist()
    tile_req, tile_q0, dec_req, dec_tok, max_decode_kv = cut_attention_work(
        cu, kv, ctx.num_requests, queries_per_tile, split_decodes)
    work = AttentionWork()
    work.num_tiles, work.num_decode, work.max_decode_kv = len(tile_req), len(dec_req), max_decode_kv
    packed = torch.tensor(tile_req + tile_q0 + dec_req + dec_tok, dtype=torch.int32).to(device)
    nt, nd = work.num_tiles, work.num_decode
    work.tile_req, work.tile_q0 = packed[:nt], packed[nt:2 * nt]
    work.dec_req, work.dec_tok = packed[2 * nt:2 * nt + nd], packed[2 * nt + nd:]
    if cache is not None:
        cache[key] = work
    return work


def timeline_read(reset=True):
    """The records of a TINYSERVE_TIMELINE=1 build, from every loaded library, as a numpy structured
    array sorted by time: ns, sm, tag (0 block started, 1 its wait for the predecessor returned,
    2 and 3 marks of the kernel itself), grid and block indices, threads per block."""
    import numpy as np
    dtype = np.dtype([("ns", "<u8"), ("sm", "<i4"), ("tag", "<i4"), ("grid", "<i4", 3), ("block", "<i4", 3),
                      ("threads", "<i4"), ("pad", "<i4")])
    chunks = []
    for lib in build.loaded_units():
        if not hasattr(lib, "ts_timeline_read"):
            continue
        buf = np.zeros(1 << 17, dtype=dtype)
        n = lib.ts_timeline_read(ctypes.c_void_p(buf.ctypes.data), c_int(len(buf)), c_int(1 if reset else 0))
        if n < 0:
            raise RuntimeError("reading the kernel timeline failed")
        chunks.append(buf[:n])
    if not chunks:
        raise RuntimeError("no loaded library records a timeline: set TINYSERVE_TIMELINE=1 before the first kernel is built")
    out = np.concatenate(chunks)
    return out[np.argsort(out["ns"], kind="stable")]


def _tma_pages(k_cache, v_cache):
    """The page count that lets the decode kernel fetch whole pages by TMA, or 0 where the caches
    are not plain [pages, kv heads, page, head] blocks of memory."""
    return k_cache.shape[0] if k_cache.is_contiguous() and v_cache.is_contiguous() else 0


def decode_splits(num_requests, max_kv_len, num_heads, num_kv_heads):
    """Key ranges for the tensor-core decode kernel: as many as fit in one wave of blocks (two
    per SM), with at least two tiles of 64 keys per range."""
    blocks = num_kv_heads * -(-(num_heads // num_kv_heads) // 16) * num_requests
    return max(1, min(2 * num_sms() // blocks, max_kv_len // 128, 32))


def _decode_listed(q, out, k_cache, v_cache, view, ctx, scale, window, work):
    """The one-token requests of a mixed batch, by the tensor-core decode kernel."""
    T, H, D = q.shape
    Hkv = k_cache.shape[1]
    n = work.num_decode
    num_splits = decode_splits(n, work.max_decode_kv, H, Hkv)
    part_o = part_ml = None
    cluster = 1 < num_splits <= CLUSTER_MERGE_MAX_SPLITS
    if num_splits > 1 and not cluster:
        part_o = torch.empty(n * H * num_splits * D, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n * H * num_splits * 2, dtype=torch.float32, device=q.device)
    lib = _attention_mma(D)
    _check(lib, lib.ts_paged_attention_mma(
        _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(view.block_table), _ptr(ctx.cu_q),
        _ptr(ctx.kv_lens), c_int(T), c_int(ctx.num_requests), c_int(1), c_int(H), c_int(Hkv),
        c_int(view.page_size), c_int(view.block_table.stride(0)), c_float(scale), c_int(window),
        c_int(num_splits), _ptr(part_o), _ptr(part_ml), c_int(2 if cluster else 1), _ptr(work.dec_req),
        _ptr(work.dec_tok), c_int(n), c_int(0), c_int(_tma_pages(k_cache, v_cache)), _stream()),
        2 if num_splits > 1 and not cluster else 1)


def attention_backend(dtype, head_dim, page_size=16) -> str:
    """Which kernels attend for this element type and head size: "tcgen05" (prefill on the
    tcgen05 kernel, decode on the mma.sync decode kernel), "mma" (both on the mma.sync kernels) or
    "simt" (the 32-bit kernel: float32, and bfloat16 heads wider than MMA_MAX_HEAD_DIM)."""
    if dtype != torch.bfloat16 or head_dim > MMA_MAX_HEAD_DIM or head_dim not in SUPPORTED_HEAD_DIMS:
        return "simt"
    if head_dim in TCGEN05_HEAD_DIMS and 8 <= page_size <= 128 and page_size & (page_size - 1) == 0:
        return "tcgen05"
    return "mma"


def prefill_tile_queries(dtype, num_heads, num_kv_heads, head_dim, page_size=16) -> int:
    """Queries per block of the prefill kernel that ``attention_backend`` names (0: the kernel
    takes no work list)."""
    group = num_heads // num_kv_heads
    backend = attention_backend(dtype, head_dim, page_size)
    if backend == "tcgen05":
        return 2 * (128 // group if group < 128 else 1)      # two query tiles of 128 rows a block
    if backend == "mma":
        return MMA_PREFILL_ROWS // group if group < MMA_PREFILL_ROWS else 1
    return 0


def paged_attention(q, k_cache, v_cache, view, ctx, scale, window=0, num_splits=None, backend=None):
    """Attention of this step's queries over their requests' cached keys and values.
    q [T, H, D]; caches [pages, Hkv, page_size, D]; ``view`` a GroupView; ``ctx`` gives cu_q,
    kv_lens and the batch's maxima.  bfloat16 runs on the tensor cores (a decode kernel when
    every request brings one token, else a prefill kernel); float32 on the 32-bit kernel.
    ``backend`` overrides ``attention_backend`` (tests run the slower kernels at every size)."""
    _cuda(q, k_cache, v_cache)
    T, H, D = q.shape
    Hkv = k_cache.shape[1]
    page = view.page_size
    chosen = attention_backend(q.dtype, D, page)
    if backend is not None and backend != chosen:
        if q.dtype != torch.bfloat16 or (backend == "tcgen05") or (backend == "mma" and chosen == "simt"):
            raise ValueError(f"attention backend {backend!r} does not take {q.dtype}, head size {D}, pages of {page}")
        chosen = backend
    if chosen == "tcgen05" and not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        chosen = "mma"
    mma = chosen in ("tcgen05", "mma")
    decode = mma and ctx.max_q_len == 1
    if chosen == "tcgen05" and not decode:
        out = torch.empty_like(q)
        lib = _attention_tcgen05(D)
        tile_queries = prefill_tile_queries(q.dtype, H, Hkv, D, page)
        work = attention_work(ctx, tile_queries, q.device)
        if work.num_decode:
            _decode_listed(q, out, k_cache, v_cache, view, ctx, scale, window, work)
        if work.num_tiles:
            _check(lib, lib.ts_paged_attention_tcgen05(
                _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(view.block_table), _ptr(ctx.cu_q),
                _ptr(ctx.kv_lens), c_int(T), c_int(ctx.num_requests), c_int(ctx.max_q_len), c_int(H), c_int(Hkv),
                c_int(k_cache.shape[0]), c_int(page), c_int(view.block_table.stride(0)), c_float(scale),
                c_int(window), _ptr(work.tile_req), _ptr(work.tile_q0), c_int(work.num_tiles),
                c_int(tile_queries), _stream()))
        return out
    if num_splits is None:
        if decode:
            num_splits = decode_splits(ctx.num_requests, ctx.max_kv_len, H, Hkv)
        elif mma:
            num_splits = 1
        else:
            num_splits = attention_splits(ctx.num_requests, ctx.max_q_len, ctx.max_kv_len, H, Hkv)
    if mma and not decode:
        num_splits = 1
    out = torch.empty_like(q)
    part_o = part_ml = None
    cluster = mma and decode and 1 < num_splits <= CLUSTER_MERGE_MAX_SPLITS
    if num_splits > 1 and not cluster:
        part_o = torch.empty(T * H * num_splits * D, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(T * H * num_splits * 2, dtype=torch.float32, device=q.device)
    launches = 2 if num_splits > 1 and not cluster else 1
    if mma:
        lib = _attention_mma(D)
        tile_req = tile_q0 = None
        num_tiles = tile_queries = 0
        if not decode:
            group = H // Hkv
            tile_queries = MMA_PREFILL_ROWS // group if group < MMA_PREFILL_ROWS else 1
            work = attention_work(ctx, tile_queries, q.device)
            if work.num_decode:
                _decode_listed(q, out, k_cache, v_cache, view, ctx, scale, window, work)
            if not work.num_tiles:
                return out
            tile_req, tile_q0, num_tiles = work.tile_req, work.tile_q0, work.num_tiles
        _check(lib, lib.ts_paged_attention_mma(
            _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(view.block_table), _ptr(ctx.cu_q),
            _ptr(ctx.kv_lens), c_int(T), c_int(ctx.num_requests), c_int(ctx.max_q_len), c_int(H),
            c_int(Hkv), c_int(view.page_size), c_int(view.block_table.stride(0)), c_float(scale),
            c_int(window), c_int(num_splits), _ptr(part_o), _ptr(part_ml),
            c_int((2 if cluster else 1) if decode else 0), _ptr(tile_req), _ptr(tile_q0), c_int(num_tiles), c_int(tile_queries),
            c_int(_tma_pages(k_cache, v_cache)), _stream()), launches)
        return out
    lib = _attention(D)
    _check(lib, lib.ts_paged_attention(
        c_int(_dt(q)), _ptr(q), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(view.block_table),
        _ptr(ctx.cu_q), _ptr(ctx.kv_lens), c_int(T), c_int(ctx.num_requests), c_int(ctx.max_q_len),
        c_int(H), c_int(Hkv), c_int(view.page_size), c_int(view.block_table.stride(0)),
        c_float(scale), c_int(window), c_int(num_splits), _ptr(part_o), _ptr(part_ml), _stream()),
        launches)
    return out


def attention_from_qkv(qkv, positions, num_heads, num_kv_heads, head_dim, rotary, q_weight, k_weight, eps,
                       k_cache, v_cache, view, ctx, scale, window=0, write_cache=True, fused=True):
    """Per-head norm of q and k, rotary encoding, cache write of k and v, attention over the cache:
    qkv [T, (H + 2 Hkv) * D] (a tensor, or the SplitPartials of the projection) -> [T, H, D].
    Two kernels (qk_norm_rope_kvwrite, paged_attention), or, when every request brings one token
    (bfloat16, full-width rotary with the (j, j + D/2) pairing), the decode kernel alone: it makes
    its query rows and the newest key and value itself (one kernel fewer per layer; ``fused``
    False keeps the two kernels, for comparison)."""
    dtype = qkv.dtype
    H, Hkv, D = num_heads, num_kv_heads, head_dim
    plain = isinstance(qkv, torch.Tensor)
    # (up to FUSED_MAX_TOKENS requests: measured, at 64 the separate kernel is 4 % of the step faster)
    fused = (fused and write_cache and dtype == torch.bfloat16 and ctx.max_q_len == 1
             and qkv.shape[0] <= FUSED_MAX_TOKENS
             and D in SUPPORTED_HEAD_DIMS and D <= MMA_MAX_HEAD_DIM
             and rotary is not None and rotary.rotary_dim == D and not rotary.interleaved
             and (q_weight is None) == (k_weight is None)
             and k_cache is not None and k_cache.dtype == torch.bfloat16
             and (isinstance(qkv, SplitPartials) or (plain and qkv.is_contiguous()))
             and (q_weight is None or q_weight.dtype == k_weight.dtype))
    if not fused:
        q = qk_norm_rope_kvwrite(qkv, positions, H, Hkv, D, rotary=rotary, q_weight=q_weight, k_weight=k_weight,
                                 eps=eps, k_cache=k_cache, v_cache=v_cache,
                                 slot_mapping=view.slot_mapping if write_cache else None, page_size=view.page_size)
        return paged_attention(q, k_cache, v_cache, view, ctx, scale, window)
    T = qkv.shape[0]
    if qkv.shape[1] != (H + 2 * Hkv) * D:
        raise ValueError("qkv must be [T, (H + 2 Hkv) * D]")
    parts = _NO_PARTIALS if plain else qkv.args()
    _cuda(qkv if plain else None, positions, k_cache, v_cache, view.slot_mapping, view.block_table, rotary.cos, rotary.sin)
    out = torch.empty(T, H, D, dtype=dtype, device=qkv.device)
    num_splits = decode_splits(ctx.num_requests, ctx.max_kv_len, H, Hkv)
    cluster = 1 < num_splits <= CLUSTER_MERGE_MAX_SPLITS
    part_o = part_ml = None
    if num_splits > 1 and not cluster:
        part_o = torch.empty(T * H * num_splits * D, dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty(T * H * num_splits * 2, dtype=torch.float32, device=qkv.device)
    lib = _attention_mma(D)
    _check(lib, lib.ts_paged_attention_mma_from_qkv(
        _ptr(qkv) if plain else None, *parts, _ptr(positions), _ptr(view.slot_mapping), _ptr(rotary.cos),
        _ptr(rotary.sin), _ptr(q_weight), _ptr(k_weight), c_int(_vec_flag(q_weight, dtype) if q_weight is not None else 0),
        c_float(eps), _ptr(out), _ptr(k_cache), _ptr(v_cache), _ptr(view.block_table), _ptr(ctx.cu_q),
        _ptr(ctx.kv_lens), c_int(T), c_int(ctx.num_requests), c_int(H), c_int(Hkv), c_int(view.page_size),
        c_int(view.block_table.stride(0)), c_float(scale), c_int(window), c_int(num_splits), _ptr(part_o),
        _ptr(part_ml), c_int(2 if cluster else 1), c_int(_tma_pages(k_cache, v_cache)), _stream()),
        2 if num_splits > 1 and not cluster else 1)
    return out


def linear(x, weight, bias=None, out_float32=False, allow_partials=False, allow_pending=False):
    """x [M, K] @ weight[N, K]^T (+ bias).  float32 operands: this package's 32-bit FMA kernel
    (no tensor cores, no reduced precision).  bfloat16 operands: this package's TMA + tcgen05
    kernel for up to TCGEN05_MAX_TOKENS rows (K and the leading dimensions multiples of 8), cuBLAS
    through torch above that, as in tinyserve (serve.py:828-829).  With ``allow_partials`` the
    result may be a SplitPartials (the caller hands it to add_rmsnorm, qk_norm_rope_kvwrite, or
    calls materialize); with ``allow_pending`` a PendingProduct (for add_rmsnorm, or materialize).
    x may be the ScaledRows that add_rmsnorm returned."""
    scale = None
    if isinstance(x, ScaledRows):
        scale, x = x, x.data
    _cuda(x, weight, bias)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or x.dtype != weight.dtype:
        raise ValueError(f"linear: x {tuple(x.shape)} {x.dtype} does not fit weight {tuple(weight.shape)} {weight.dtype}")
    if bias is not None and tuple(bias.shape) != (N,):
        raise ValueError(f"linear: bias {tuple(bias.shape)} does not fit {N} outputs")
    x = materialize(x)
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and M >= PAIR_MIN_TOKENS and _pair_ok(x, weight):
        if allow_pending and scale is None and bias is None and not out_float32:
            return PendingProduct(x, weight, wide=True)
        return _linear_pair(x, weight, out_float32, bias=bias, scale=scale)
    if x.dtype == torch.bfloat16 and _tcgen05_ok(x, weight) and (scale is None or M <= FUSED_MAX_TOKENS):
        if bias is not None:
            if scale is not None:
                x, scale = scale.materialize(), None
            return _linear_tcgen05(x, weight, out_float32, bias=bias)
        if allow_pending and scale is None and not out_float32 and M <= FUSED_MAX_TOKENS:
            return PendingProduct(x, weight)
        if (allow_partials or allow_pending) and not out_float32 \
                and gemm_splits(x.shape[0], weight.shape[0], x.shape[1], partials=True) > 1:
            return _linear_tcgen05(x, weight, False, partials_only=True, scale=scale)
        return _linear_tcgen05(x, weight, out_float32, scale=scale)
    if scale is not None:
        x = scale.materialize()
    if x.dtype == torch.bfloat16:
        # a plain library product (and its bias epilogue), as in tinyserve
        if bias is not None:
            out = torch.addmm(bias.to(torch.bfloat16), x, weight.t())
            return out.float() if out_float32 else out
        if out_float32:
            return torch.mm(x, weight.t(), out_dtype=torch.float32)
        return torch.mm(x, weight.t())
    return _linear_simt(x, weight, bias, out_float32)


def _linear_simt(x, weight, bias=None, out_float32=False):
    """The 32-bit FMA product (float32 operands; it takes bfloat16 operands too)."""
    M, K = x.shape
    N = weight.shape[0]
    out_dtype = torch.float32 if out_float32 else x.dtype
    out = torch.empty(M, N, dtype=out_dtype, device=x.device)
    if x.stride(1) != 1 or weight.stride(1) != 1:
        raise ValueError("linear: operands must be contiguous along K")
    if bias is not None and bias.dtype != x.dtype:
        bias = bias.to(x.dtype)
    lib = _gemm()
    _check(lib, lib.ts_gemm_simt(c_int(_dt(x)), c_int(_DTYPE[out_dtype]), _ptr(x), _ptr(weight),
                                 _ptr(bias), _ptr(out), c_int(M), c_int(N), c_int(K),
                                 c_longlong(x.stride(0)), c_longlong(weight.stride(0)),
                                 c_longlong(N), _stream()))
    return out


def sample(logits, temperature, stream_ids, steps, seed, top_k=None, top_p=None, slot_tokens=None,
           slots=None):
    """One token per row of float32 logits.  temperature float32 [B] (0 = argmax); stream_ids
    int64 [B] and steps int32 [B] select the noise; top_k int32 [B], top_p float32 [B] optional.
    With ``slot_tokens`` (int32 [slots]) and ``slots`` (int32 [B]) row i's token is also stored
    at slot_tokens[slots[i]], for the next step's embedding lookup."""
    _cuda(logits, temperature, stream_ids, steps, top_k, top_p, slot_tokens, slots)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise TypeError("sample: logits must be float32 rows")
    B, V = logits.shape
    out = torch.empty(B, dtype=torch.int32, device=logits.device)
    lib = _sampler()
    _check(lib, lib.ts_sample(_ptr(logits), c_longlong(logits.stride(0)), c_int(B), c_int(V),
                              _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(stream_ids),
                              _ptr(steps), c_ulonglong(seed & (2 ** 64 - 1)), _ptr(out),
                              _ptr(slot_tokens), _ptr(slots), _stream()))
    return out


def apply_repetition_penalty(logits, rows, ids, penalty):
    """In place: rows int32 [R] of logits; ids int32 [R, n] distinct recent tokens (-1 = none);
    penalty float32 [R]."""
    _cuda(logits, rows, ids, penalty)
    lib = _sampler()
    _check(lib, lib.ts_apply_repetition_penalty(
        _ptr(logits), c_longlong(logits.stride(0)), c_int(logits.shape[1]), _ptr(rows), _ptr(ids),
        c_int(rows.shape[0]), c_int(ids.shape[1]), _ptr(penalty), _stream()))
    return logits
