"""The step function: run a batch of (request, its next tokens) from the cache.

``ModelRunner`` owns the model, the device cache, the host cache manager and the
persistent input buffers.  ``step(entries)`` packs the entries (whole prompts,
portions of prompts and single decoded tokens, cut anywhere) into one batch, uploads
it with one copy, runs only those tokens through the model and returns 32-bit logits
at the wanted places.  Nothing here samples, schedules or decides who runs.

tinyserve's counterpart is ``ModelRunner`` (serve.py:1604-2114): ``_pack`` builds ids,
positions, slots, query starts, lengths and the block table per request
(serve.py:1853-1875), ``_upload`` copies them into persistent buffers
(serve.py:1910-1915) and decode-only batches replay captured graphs
(serve.py:1969-2053).  It always returns the last row of every request
(serve.py:1875, 2077); here the caller says which rows it wants.  Here every state slot keeps
its request's block-table row on the device and a step uploads only the entries that changed;
the attention work lists of a step with prompt portions travel in the same copy."""
from __future__ import annotations

import numpy as np
import torch

from ..cache.device import DeviceCache
from ..cache.manager import CacheError, CacheManager, GroupSpec
from ..config.engine_config import EngineConfig
from ..config.registry import load_model_config
from ..kernels import ops
from ..weights import fill_random_on_device, load_weights
from ..parts.model import build_model
from .batch import GroupView, StepContext, StepEntry

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


PENDING = -1     # a token id that is still on the device (see ModelRunner.slot_tokens)


# Token counts for which steps that hold prompt portions are captured as graphs: above the
# largest a step is busy enough with arithmetic that its launches hardly matter, and runs eagerly
# (tinyserve's buckets are every 16 tokens up to 512, serve.py:1951-1962).
MIXED_GRAPH_TOKENS = (16, 32, 48, 64, 96, 128, 192, 256, 384, 512)
MIXED_GRAPHS_KEPT = 16           # captured shapes kept; the one replayed longest ago goes first
MIXED_GRAPH_SIGHTINGS = 2        # steps of a shape that run eagerly before the shape is captured


class Prepared:
    """A packed step that waits for its launch.  ``graph``: the captured decode graph it
    replays; ``mixed``: the captured shape (tokens, requests, logit rows, context bound) it was padded to."""

    def __init__(self, entries, ctx, graph, buf, mixed=None):
        self.entries, self.ctx, self.graph, self.buf, self.mixed = entries, ctx, graph, buf, mixed


class _Runtime:
    """What parts may ask of the engine when they build their constants (``Part.prepare``)."""

    def __init__(self, device, max_positions, dtype):
        self.device, self.max_positions, self.dtype = device, max_positions, dtype
        self.shared: dict = {}       # tables that several parts of this engine share


class ModelRunner:
    def __init__(self, cfg: EngineConfig, model_config=None, random_weights=False, verbose=False):
        ops.require_device(cfg.device)
        self.cfg = cfg
        self.device = torch.device(cfg.device)
        self.dtype = _TORCH_DTYPES[cfg.dtype]
        self.model_config = model_config or load_model_config(cfg.model)
        self.model = build_model(self.model_config)
        if random_weights:
            self.weight_bytes = fill_random_on_device(self.model, self.dtype, self.device, cfg.seed)
        else:
            self.weight_bytes = load_weights(self.model, cfg.model, self.dtype, self.device)
        self.model.prepare(_Runtime(self.device, cfg.max_model_len, self.dtype))
        self.page_size = cfg.block_size
        self.max_blocks = -(-cfg.max_model_len // self.page_size)
        self.num_pages = self._size_cache()
        self.device_cache = DeviceCache(self.model, self.num_pages, self.page_size,
                                        cfg.max_num_seqs, self.dtype, self.device)
        groups = [GroupSpec(s.kind, s.window) for s in self.model.cache_groups]
        self.manager = CacheManager(groups, self.num_pages, self.page_size, cfg.max_num_seqs)
        self._make_buffers()
        self.graphs: dict = {}
        # graphs of steps with prompt portions, captured when a shape comes up the second time
        self.mixed_graphs: dict = {}
        self.mixed_graphs_enabled = False
        self.mixed_graph_replays = 0
        self._graph_pool = None
        self._capture_stream = None
        self.kernel_launches = 0
        self.last_upload_bytes = 0
        if verbose:
            print(f"[tinyserve_b200] weights {self.weight_bytes / 2**30:.2f} GiB, "
                  f"{self.num_pages - 1} pages of {self.page_size} tokens per cache group "
                  f"({len(groups)} group(s))", flush=True)

    # ------------------------------------------------------------------ set-up
    def _size_cache(self) -> int:
        cfg = self.cfg
        cap = cfg.max_num_seqs * self.max_blocks + 1
        if cfg.num_blocks:
            return cfg.num_blocks + 1 if cfg.num_blocks + 1 <= cap else cap
        per_page = sum(DeviceCache.bytes_per_page(self.model, self.page_size,
                                                  torch.empty((), dtype=self.dtype).element_size()))
        if per_page == 0:
            return 2
        free, total = torch.cuda.mem_get_info(self.device)
        # leave room for activations of a full step and for logits
        reserve = cfg.max_num_batched_tokens * self._activation_bytes_per_token() + \
            cfg.max_num_seqs * self.model.vocab_size * 8 + (1 << 30)
        budget = min(total * cfg.gpu_memory_utilization - (total - free), free) - reserve
        pages = int(budget // per_page)
        if (pages - 1) * self.page_size < cfg.max_model_len:
            raise CacheError(
                f"the cache would hold {max(0, pages - 1) * self.page_size} tokens, fewer than "
                f"max_model_len {cfg.max_model_len}: lower max_model_len or raise gpu_memory_utilization")
        return min(pages, cap)

    def _activation_bytes_per_token(self) -> int:
        widest = self.model.hidden_size
        for block in self.model.blocks:
            for part in block.named_parts():
                for spec in part.param_specs().values():
                    if len(spec.shape) == 2:
                        widest = max(widest, spec.shape[0])
        return 4 * widest * 4

    def _make_buffers(self):
        """One staging layout for everything a step uploads: a header, the per-request and per-token
        arrays, the attention work lists of the tile sizes the mixers announce, and at the end the
        block-table changes (pairs of flat index and page), of which only the used part is copied."""
        cfg = self.cfg
        N, S = cfg.max_num_batched_tokens, cfg.max_num_seqs
        G = len(self.model.cache_groups)
        self._tile_sizes = sorted({q for block in self.model.blocks
                                   for q in [block.mixer.work_tile_queries(self.dtype, self.page_size)] if q > 0})
        # (one request more than max_num_seqs: a captured mixed shape always ends in an empty one)
        sizes = [("meta", 4), ("cu_q", S + 2), ("kv_lens", S + 1), ("state_slots", S + 1), ("fresh", S + 1),
                 ("token_ids", N), ("positions", N), ("logit_rows", N)]
        for g in range(G):
            sizes.append((f"slot_mapping{g}", N))
        for q in self._tile_sizes:
            sizes += [(f"tile_req{q}", N // q + S + 1), (f"tile_q0{q}", N // q + S + 1)]
        if self._tile_sizes:
            sizes += [("dec_req", S + 1), ("dec_tok", S + 1)]
        self._offsets, total = {}, 0
        for name, n in sizes:
            self._offsets[name] = (total, n)
            total += (n + 3) // 4 * 4
        self._pairs_at = total
        self._pairs_capacity = max(1, G * S * self.max_blocks)
        total += 2 * self._pairs_capacity
        # two staging buffers: a step is packed while the copy of the one before may be pending
        self._hosts = [torch.zeros(total, dtype=torch.int32).pin_memory() if self.device.type == "cuda"
                       else torch.zeros(total, dtype=torch.int32) for _ in range(2)]
        self._hosts_np = [h.numpy() for h in self._hosts]
        self._used = [total, total]      # words of each staging buffer that the packed step uses
        self._copied = [None, None]      # event after the last copy out of each staging buffer
        self._next_buf = 0
        self._dev = torch.zeros(total, dtype=torch.int32, device=self.device)
        # block tables: a resident row per state slot (and a spare row of null pages), the rows of the
        # step's requests gathered from them
        self._resident_tables = torch.zeros(max(G, 1), S + 1, self.max_blocks, dtype=torch.int32, device=self.device)
        self._step_tables = torch.zeros(max(G, 1), S + 1, self.max_blocks, dtype=torch.int32, device=self.device)
        # last sampled token of every state slot (one spare entry for rows nobody waits for)
        self.slot_tokens = torch.zeros(S + 1, dtype=torch.int32, device=self.device)

    def _seg(self, buf, name, n=None):
        off, cap = self._offsets[name]
        return buf[off:off + (cap if n is None else n)]

    # ------------------------------------------------------------------ packing
    def _pack(self, entries, buf=0, pad_requests=0, pad_tokens=0, shape=None):
        """Fill host staging buffer ``buf``; returns a StepContext without device work.
        ``shape`` = (tokens, requests, logit rows, context bound) packs a step with prompt portions as the
        captured shape of that size: token rows and requests padded, the attention work lists
        filled up to their capacity with entries that name the last (empty) request, and the
        context's maxima set to the shape's, so that every launch has the shape's grid."""
        cfg, mgr, ps = self.cfg, self.manager, self.page_size
        B = len(entries)
        T = sum(len(e.tokens) for e in entries)
        if B == 0 or T == 0:
            raise ValueError("a step needs at least one token")
        if shape is not None:
            pad_tokens, pad_requests = shape[0], shape[1]
        Bp, Tp = max(B, pad_requests), max(T, pad_tokens)
        if Tp > cfg.max_num_batched_tokens:
            raise ValueError(f"{Tp} tokens in one step, max_num_batched_tokens is {cfg.max_num_batched_tokens}")
        if B > cfg.max_num_seqs or Bp > cfg.max_num_seqs + (shape is not None):
            raise ValueError(f"{Bp} requests in one step, max_num_seqs is {cfg.max_num_seqs}")
        h = self._hosts_np[buf]
        seg = lambda name, n=None: self._seg(h, name, n)
        ids, pos, rows = seg("token_ids"), seg("positions"), seg("logit_rows")
        cu_q, kv_lens, slots, fresh = seg("cu_q"), seg("kv_lens"), seg("state_slots"), seg("fresh")
        G, S, MB = len(self.model.cache_groups), cfg.max_num_seqs, self.max_blocks
        slot_maps = [seg(f"slot_mapping{g}") for g in range(G)]
        pairs = h[self._pairs_at:]
        num_pairs, receipts = 0, []
        t = w = 0
        max_q = max_kv = 0
        cu_q[0] = 0
        for b, e in enumerate(entries):
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.rid!r} brings no token")
            start = mgr.num_computed(e.rid)
            if start + n > cfg.max_model_len:
                raise ValueError(f"request {e.rid!r} would hold {start + n} tokens, max_model_len is {cfg.max_model_len}")
            if any(mgr.pages_needed(e.rid, n)) and not mgr.allocate(e.rid, n):
                raise CacheError(f"no cache pages left for request {e.rid!r}")
            slot = mgr.slot(e.rid)
            for g in range(G):
                # only what the device's copy of the request's row lacks travels
                changes, receipt = mgr.table_updates(e.rid, g)
                if changes:
                    base = (g * (S + 1) + slot) * MB
                    for index, page in changes:
                        pairs[2 * num_pairs] = base + index
                        pairs[2 * num_pairs + 1] = page
                        num_pairs += 1
                    receipts.append(receipt)
            if n == 1:
                # a decoded token: scalars, no temporaries
                tok = e.tokens[0]
                ids[t] = tok if tok >= 0 else -1 - slot                # pending: read on the device
                pos[t] = start
                for g in range(G):
                    slot_maps[g][t] = mgr.block_table(e.rid, g)[start // ps] * ps + start % ps
            else:
                if min(e.tokens) < 0:
                    raise ValueError(f"request {e.rid!r}: only a single decoded token may be pending")
                ids[t:t + n] = e.tokens
                pos[t:t + n] = np.arange(start, start + n, dtype=np.int32)
                p = np.arange(start, start + n)
                for g in range(G):
                    pages = np.asarray(mgr.block_table(e.rid, g), dtype=np.int64)
                    slot_maps[g][t:t + n] = pages[p // ps] * ps + p % ps
            for j in e.want:
                if not 0 <= j < n:
                    raise ValueError(f"request {e.rid!r} wants place {j} of {n} tokens")
                rows[w] = t + j
                w += 1
            t += n
            cu_q[b + 1] = t
            kv_lens[b] = start + n
            slots[b] = slot
            fresh[b] = 1 if start == 0 else 0
            max_q, max_kv = max(max_q, n), max(max_kv, start + n)
        # padding of a captured shape: token rows that write nowhere, requests without tokens (their
        # block-table rows are the spare row of null pages)
        if Tp > T:
            ids[T:Tp] = 0
            pos[T:Tp] = 0
            for g in range(G):
                slot_maps[g][T:Tp] = -1
        for b in range(B, Bp):
            cu_q[b + 1] = T
            kv_lens[b] = 0
            slots[b] = S
            fresh[b] = 0
        seg("meta")[0] = num_pairs
        self._used[buf] = self._pairs_at + 2 * num_pairs
        ctx = StepContext()
        ctx.num_tokens, ctx.num_requests = Tp, Bp
        ctx.max_q_len, ctx.max_kv_len = max_q, max_kv
        ctx.decode_only = max_q == 1
        ctx.num_logit_rows = w
        ctx.host = {"real_tokens": T, "real_requests": B, "cu_q": cu_q[:Bp + 1].tolist(),
                    "kv_lens": kv_lens[:Bp].tolist(), "state_slots": slots[:Bp].tolist(),
                    "fresh": fresh[:Bp].tolist(), "table_receipts": receipts, "work": {}}
        if not ctx.decode_only:
            # attention work lists of the step, for the block sizes the mixers announced
            for q in self._tile_sizes:
                tile_req, tile_q0, dec_req, dec_tok, longest = ops.cut_attention_work(
                    ctx.host["cu_q"], ctx.host["kv_lens"], Bp, q)
                nt, nd = len(tile_req), len(dec_req)
                seg(f"tile_req{q}")[:nt] = tile_req
                seg(f"tile_q0{q}")[:nt] = tile_q0
                seg("dec_req")[:nd] = dec_req
                seg("dec_tok")[:nd] = dec_tok
                if shape is not None:
                    # the captured shape's lists: what is left of them names the empty last request
                    cap_t, cap_d = self._mixed_tiles(Tp, Bp, q), Bp
                    seg(f"tile_req{q}")[nt:cap_t] = Bp - 1
                    seg(f"tile_q0{q}")[nt:cap_t] = 0
                    seg("dec_req")[nd:cap_d] = Bp - 1
                    seg("dec_tok")[nd:cap_d] = -1
                    nt, nd, longest = cap_t, cap_d, shape[3]
                ctx.host["work"][q] = (nt, nd, longest)
        if shape is not None:
            assert w <= shape[2] and B < Bp
            rows[w:shape[2]] = 0
            ctx.num_logit_rows = shape[2]
            ctx.max_q_len, ctx.max_kv_len = Tp, shape[3]
        return ctx

    @staticmethod
    def _mixed_tiles(tokens, requests, queries_per_tile):
        """Most blocks of ``queries_per_tile`` queries that ``tokens`` tokens of up to ``requests``
        requests are cut into (every request may end in a block that is not full)."""
        return tokens // queries_per_tile + min(requests, tokens // 2 + 1)

    def _bind_device_views(self, ctx):
        d = self._dev
        T, B = ctx.num_tokens, ctx.num_requests
        ctx.token_ids = self._seg(d, "token_ids", T)
        ctx.positions = self._seg(d, "positions", T)
        ctx.logit_rows = self._seg(d, "logit_rows", ctx.num_logit_rows)
        ctx.cu_q = self._seg(d, "cu_q", B + 1)
        ctx.kv_lens = self._seg(d, "kv_lens", B)
        ctx.state_slots = self._seg(d, "state_slots", B)
        ctx.fresh = self._seg(d, "fresh", B)
        ctx.groups = []
        for g in range(len(self.model.cache_groups)):
            ctx.groups.append(GroupView(self.page_size, self.max_blocks, self._seg(d, f"slot_mapping{g}", T),
                                        self._step_tables[g, :B], self.num_pages))
        for q, (nt, nd, longest) in ctx.host.get("work", {}).items():
            work = ops.AttentionWork()
            work.num_tiles, work.num_decode, work.max_decode_kv = nt, nd, longest
            work.tile_req, work.tile_q0 = self._seg(d, f"tile_req{q}", nt), self._seg(d, f"tile_q0{q}", nt)
            work.dec_req, work.dec_tok = self._seg(d, "dec_req", nd), self._seg(d, "dec_tok", nd)
            ctx.tile_cache[(q, True)] = work
        ctx.device_cache = self.device_cache
        ctx.dtype = self.dtype
        ctx.slot_tokens = self.slot_tokens
        return ctx

    def _copy_in(self, buf=0):
        """One copy: the used part of staging buffer ``buf``."""
        used = self._used[buf]
        self._dev[:used].copy_(self._hosts[buf][:used], non_blocking=True)
        self.last_upload_bytes = used * 4

    def _tables_step(self, num_requests=None):
        """The step's block-table changes go into the resident rows; the rows of its requests are
        gathered into the tables that the attention kernels index by request."""
        if not len(self.model.cache_groups):
            return
        pairs = self._dev[self._pairs_at:].view(self._pairs_capacity, 2)
        B = num_requests if num_requests is not None else self.cfg.max_num_seqs
        ops.block_tables_step(self._resident_tables, pairs, self._seg(self._dev, "meta", 1), self._step_tables,
                              self._seg(self._dev, "state_slots"), B)

    def _upload(self, buf=0, num_requests=None):
        self._copy_in(buf)
        with ops.stream_scope():
            self._tables_step(num_requests)

    def _check_host(self, ctx, buf):
        """The host half of the index check: every index buffer of the packed step against the size
        of what it indexes, before anything is uploaded."""
        h = self._hosts_np[buf]
        seg = lambda name, n: self._seg(h, name, n)
        T, B, cfg = ctx.num_tokens, ctx.num_requests, self.cfg
        S, vocab = cfg.max_num_seqs, self.model.vocab_size
        ids, pos, cu, kv = seg("token_ids", T), seg("positions", T), seg("cu_q", B + 1), seg("kv_lens", B)
        problems = []
        if ((ids >= vocab) | (ids < -S)).any():
            problems.append(f"a token id outside [0, {vocab}) that names no state slot")
        if ((pos < 0) | (pos >= cfg.max_model_len)).any():
            problems.append(f"a position outside [0, {cfg.max_model_len})")
        rows = seg("logit_rows", ctx.num_logit_rows)
        if ((rows < 0) | (rows >= T)).any():
            problems.append(f"a wanted row outside the batch of {T} tokens")
        q_lens = np.diff(cu)
        if cu[0] != 0 or (q_lens < 0).any() or cu[B] > T:
            problems.append("query offsets that are not 0 .. T in ascending order")
        elif ((kv < q_lens) | (kv > cfg.max_model_len)).any():
            problems.append("a request whose length is below its new tokens or above max_model_len")
        slots = seg("state_slots", B)
        if ((slots < 0) | (slots > S)).any():               # S itself is the spare slot of padded requests
            problems.append(f"a state slot outside [0, {S}]")
        for g in range(len(self.model.cache_groups)):
            sm = seg(f"slot_mapping{g}", T)
            if ((sm < -1) | (sm >= self.num_pages * self.page_size)).any():
                problems.append(f"group {g}: a cache slot outside the pool of {self.num_pages} pages")
        n = int(self._seg(h, "meta", 1)[0])
        pairs = h[self._pairs_at:self._pairs_at + 2 * n].reshape(n, 2)
        if n < 0 or n > self._pairs_capacity or ((pairs[:, 0] < 0) | (pairs[:, 0] >= self._resident_tables.numel())).any():
            problems.append("a block-table change outside the resident tables")
        elif ((pairs[:, 1] < 0) | (pairs[:, 1] >= self.num_pages)).any():
            problems.append(f"a page number outside [0, {self.num_pages})")
        if problems:
            raise ValueError("the packed step holds " + "; ".join(problems))

    # ------------------------------------------------------------------ stepping
    def prepare(self, entries) -> Prepared:
        """Pack a step on the host (no device work).  A token id of PENDING stands for the
        request's last sampled token, which the device still holds."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        graph = self._graph_for(entries)
        mixed = self._mixed_shape_for(entries) if graph is None else None
        buf, self._next_buf = self._next_buf, self._next_buf ^ 1
        if self._copied[buf] is not None:
            # the host may run several steps ahead of the device (nobody has to read a result
            # between steps): this buffer's last copy must have left it before it is packed again
            self._copied[buf].synchronize()
        if graph is not None:
            size = graph[2]
            ctx = self._pack(entries, buf, pad_requests=size, pad_tokens=size)
            self._seg(self._hosts_np[buf], "logit_rows")[:size] = np.arange(size, dtype=np.int32)
        else:
            ctx = self._pack(entries, buf, shape=mixed)
        if self.cfg.check_indices:
            self._check_host(ctx, buf)
        return Prepared(entries, ctx, graph, buf, mixed)

    @torch.inference_mode()
    def launch(self, prep: Prepared):
        """Upload and run a prepared step; its tokens are computed afterwards."""
        # (a captured graph holds the block-table kernels itself: only the copy happens here)
        captured = prep.graph
        if prep.mixed is not None:
            captured = self._mixed_graph(prep)       # None when the shape comes up for the first time
        if captured is not None:
            self._copy_in(prep.buf)
        else:
            self._upload(prep.buf, prep.ctx.num_requests)
        for receipt in prep.ctx.host.get("table_receipts", ()):
            self.manager.table_synced(receipt)
        if self.device.type == "cuda":
            if self._copied[prep.buf] is None:
                self._copied[prep.buf] = torch.cuda.Event()
            self._copied[prep.buf].record()
        if self.device_cache.states:
            # a request that starts in this step finds its state slot zeroed, whoever held it before
            host = prep.ctx.host
            self.device_cache.zero_state([s for s, f in zip(host["state_slots"], host["fresh"]) if f])
        if captured is not None:
            graph, out, size, launches = captured
            graph.replay()
            ops.count_launches(launches)
            wanted = len(prep.entries) if prep.mixed is None else sum(len(e.want) for e in prep.entries)
            logits = out[:wanted] if wanted else None
        else:
            with ops.stream_scope():
                logits = self._forward(self._bind_device_views(prep.ctx))
            if prep.mixed is not None:
                wanted = sum(len(e.want) for e in prep.entries)
                logits = logits[:wanted] if wanted else None
        for e in prep.entries:
            if self.manager.is_live(e.rid):      # a request may have ended since it was packed
                self.manager.commit(e.rid, len(e.tokens))
        return logits

    def _forward(self, ctx):
        if self.cfg.check_indices:
            # (slot max_num_seqs is the spare one that padded requests of a captured shape name)
            ops.sanitize_step(ctx, self.model.vocab_size, self.cfg.max_model_len, self.cfg.max_model_len,
                              self.cfg.max_num_seqs + 1)
        return self.model.forward(ctx)

    def step(self, entries):
        """Run one batch.  Returns float32 logits [number of wanted places, vocab] on the
        device (None if nothing is wanted).  The entries' tokens are computed afterwards."""
        return self.launch(self.prepare(entries))

    def raise_on_device_error(self):
        """Raise ``ops.DeviceError`` if a kernel has reported that it gave up on a wait or met an
        index out of range.  Reads host memory only: call it after a synchronisation that covers
        the steps in question (reading tokens or logits back is one)."""
        ops.raise_on_device_error()

    def state_slots_on_device(self, n):
        """int32 [n] view of the state slots of the step that was launched last."""
        return self._seg(self._dev, "state_slots", n)

    # ------------------------------------------------------------------ decode graphs
    def decode_buckets(self):
        S = self.cfg.max_num_seqs
        sizes = [b for b in (1, 2, 4) if b <= S] + list(range(8, S + 1, 8))
        if S not in sizes:
            sizes.append(S)
        return sorted(set(sizes))

    def context_bounds(self):
        """Context lengths for which decode graphs are captured apart: the number of key ranges a
        decode attention launch is cut into is fixed in a captured graph, and the best number for
        a few hundred keys (a cluster of up to 8 ranges) is far from the best for 16,000."""
        bounds = [b for b in (1024, 4096, 16384, 65536) if b < self.cfg.max_model_len]
        return bounds + [self.cfg.max_model_len]

    def _graph_for(self, entries):
        if not self.graphs or not self.model.capturable:
            return None
        if any(len(e.tokens) != 1 or list(e.want) != [0] for e in entries):
            return None
        mgr = self.manager
        longest = max(mgr.num_computed(e.rid) for e in entries) + 1
        for size in self._graph_sizes:
            if size >= len(entries):
                for bound in self._graph_bounds:
                    if bound >= longest:
                        return self.graphs[(size, bound)]
                return None
        return None

    # ------------------------------------------------------------------ graphs of mixed steps
    def _mixed_shape_for(self, entries):
        """The captured shape (tokens, requests, logit rows, context bound) that a step with prompt
        portions is padded to, or None where it runs as it is: graphs are off, or the step is
        larger than the largest captured token count.  Logit rows: one per request (what serving
        asks for) or, where more are wanted, one per token."""
        if not self.mixed_graphs_enabled:
            return None
        T = sum(len(e.tokens) for e in entries)
        B = len(entries)
        tokens = next((t for t in MIXED_GRAPH_TOKENS if t >= T), None)
        if tokens is None or tokens > self.cfg.max_num_batched_tokens or B > self.cfg.max_num_seqs:
            return None
        # one request more than the step holds: the empty one that unused work-list entries name
        S = self.cfg.max_num_seqs
        requests = next((r for r in (2, 4, 8, 16, 32, 64, 128, 256, 512, 1024) if B < r <= S), S + 1)
        rows = requests if sum(len(e.want) for e in entries) <= requests else tokens
        mgr = self.manager
        longest = max(mgr.num_computed(e.rid) + len(e.tokens) for e in entries)
        bound = next((b for b in self.context_bounds() if b >= longest), None)
        return None if bound is None else (tokens, requests, rows, bound)

    def _mixed_graph(self, prep):
        """The graph of ``prep``'s captured shape.  The first steps of a shape run eagerly, in the
        padded shape (which is also the warm-up that a capture needs: a shape that comes up once
        or twice is not worth a capture); the next is captured, with its own inputs on the
        device, and replayed; later ones are replayed."""
        key = prep.mixed
        seen = self.mixed_graphs.get(key, 0)
        if isinstance(seen, int) and seen < MIXED_GRAPH_SIGHTINGS:
            self.mixed_graphs[key] = seen + 1
            return None
        if isinstance(seen, int):
            tokens, requests = key[0], key[1]
            ctx = self._bind_device_views(prep.ctx)
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            # (capture_begin / capture_end themselves: torch.cuda.graph() would also synchronise
            # the device, collect garbage and empty the allocator's cache, 30 ms a capture)
            if self._capture_stream is None:
                self._capture_stream = torch.cuda.Stream(self.device)
            self._capture_stream.wait_stream(torch.cuda.current_stream(self.device))
            try:
                with torch.cuda.stream(self._capture_stream), ops.stream_scope():
                    graph.capture_begin(pool=self._graph_pool) if self._graph_pool is not None else graph.capture_begin()
                    try:
                        self._tables_step(requests)
                        out = self._forward(ctx)
                    finally:
                        graph.capture_end()
            except torch.cuda.OutOfMemoryError:
                # no room left for another graph's buffers beside the cache: steps with portions
                # run eagerly from now on (this one too: the caller gets no graph)
                self.mixed_graphs_enabled = False
                self.mixed_graphs.pop(key, None)
                del graph
                torch.cuda.current_stream(self.device).wait_stream(self._capture_stream)
                return None
            torch.cuda.current_stream(self.device).wait_stream(self._capture_stream)
            self._graph_pool = self._graph_pool or graph.pool()
            seen = (graph, out, tokens, ops.launch_count() - before)
            captured = [k for k, v in self.mixed_graphs.items() if not isinstance(v, int)]
            if len(captured) >= MIXED_GRAPHS_KEPT:
                del self.mixed_graphs[captured[0]]
        # (the dict keeps the order of insertion: a replayed shape moves to the end)
        self.mixed_graphs.pop(key, None)
        self.mixed_graphs[key] = seen
        self.mixed_graph_replays += 1
        return seen

    @torch.inference_mode()
    def capture_decode_graphs(self, sizes=None):
        """Capture one graph per decode batch size and context bound: every request brings one
        token and wants its logits.  Smaller batches run the next larger graph with empty requests.
        A model with a part that is not ``capturable`` (it reads host-side lists of the step,
        which a replay would not refresh) is not captured: every step then runs eagerly."""
        if not self.model.capturable:
            return 0
        self.mixed_graphs_enabled = True
        sizes = sorted(sizes or self.decode_buckets(), reverse=True)
        bounds = self.context_bounds()
        pool = self._graph_pool
        dummy = "__capture__"
        self.manager.begin(dummy)
        try:
            for size, bound in [(s, b) for s in sizes for b in bounds]:
                entries = [StepEntry(dummy, [0], [0])]
                ctx = self._pack(entries, 0, pad_requests=size, pad_tokens=size)
                # captured shape: `size` requests of one token, all rows wanted
                ctx.num_logit_rows = size
                self._seg(self._hosts_np[0], "logit_rows")[:size] = np.arange(size, dtype=np.int32)
                ctx.max_kv_len = bound                # the longest context this graph is chosen for
                self._bind_device_views(ctx)
                self._copy_in(0)
                stream = torch.cuda.Stream(self.device)
                stream.wait_stream(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(stream), ops.stream_scope():
                    self._tables_step(size)
                    self._forward(ctx)                # warm-up outside capture
                torch.cuda.current_stream(self.device).wait_stream(stream)
                torch.cuda.synchronize(self.device)
                graph = torch.cuda.CUDAGraph()
                before = ops.launch_count()
                with torch.cuda.graph(graph, pool=pool), ops.stream_scope():
                    self._tables_step(size)           # every replay applies its step's block-table changes
                    out = self._forward(ctx)
                pool = self._graph_pool = pool or graph.pool()
                self.graphs[(size, bound)] = (graph, out, size, ops.launch_count() - before)
        finally:
            self.manager.free(dummy)
        self._graph_sizes = sorted({size for size, _ in self.graphs})
        self._graph_bounds = sorted({bound for _, bound in self.graphs})
        return len(self.graphs)

