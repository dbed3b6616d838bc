"""The Python entry point: ``LLM(model_dir).generate(prompts, SamplingParams(...))``.

The surface is tinyserve's ``Engine`` (serve.py:2381-2712): ``add_request``, ``step``,
``abort``, ``has_work`` and ``generate``, which adds every prompt and steps until all are
done, returning ``Output`` objects in request order (serve.py:2703-2712).  A step here is
schedule -> run the batch -> sample -> read the tokens back -> finish or go on; tinyserve
runs the host one step ahead of the device (serve.py:2509-2601); so does this engine with
``async_scheduling`` (the default): while step n runs, the tokens of step n-1 are read back and
checked, and step n+1 is scheduled and packed with placeholders for the tokens that the device
still holds (the sampler leaves each request's token at its state slot, and the embedding lookup
reads it from there).  A prompt is a string (needs the tokenizer files in the model folder) or a
list of ids."""
from __future__ import annotations

import json
import os
import time
import uuid
from dataclasses import dataclass, field
from typing import Optional

import torch

from ..config.engine_config import EngineConfig
from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .runner import PENDING, ModelRunner
from .scheduler import Request, Scheduler
from .text import Detokenizer, apply_stop_strings, load_tokenizer


@dataclass
class Output:
    """What a finished (or running) request has produced (serve.py:2295-2307)."""

    request_id: str
    text: str
    delta: str
    token_ids: list
    finished: bool
    finish_reason: Optional[str]
    num_prompt_tokens: int
    num_cached_tokens: int = 0
    logprobs: Optional[list] = None
    was_preempted: bool = False
    was_chunked_prefill: bool = False


@dataclass
class _Packed:
    """A step that is scheduled and packed on the host, not launched yet."""

    batch: list          # ScheduledRequest, in batch order
    wants: list          # per request: the step reaches its last known token, so a token is sampled
    prepared: object


@dataclass
class _Sampled:
    """A step whose tokens were sampled on the device and are on their way to the host."""

    rows: list           # (row of the logits, request, place of the token in request.token_ids)
    host: object         # pinned int32 tensor that receives the tokens
    arrived: object      # event after the copy
    raw: object          # unmodified logits, if a request wants log-probabilities


def _stop_ids(model_dir, tokenizer) -> set:
    """EOS of the tokenizer plus generation_config.json's eos_token_id (serve.py:2392-2403)."""
    ids = set()
    if tokenizer is not None and tokenizer.eos_token_id is not None:
        ids.add(tokenizer.eos_token_id)
    path = os.path.join(model_dir, "generation_config.json") if model_dir else ""
    if path and os.path.isfile(path):
        with open(path) as fh:
            eos = json.load(fh).get("eos_token_id")
        ids |= set(eos if isinstance(eos, list) else [eos])
    ids.discard(None)
    return ids


class LLM:
    def __init__(self, model: str = "", *, model_config=None, random_weights: bool = False,
                 verbose: bool = False, async_scheduling: bool = True, **engine_options):
        """``model``: a folder with config.json and safetensors.  ``engine_options`` are the
        fields of ``EngineConfig`` (dtype, max_model_len, block_size, max_num_seqs,
        max_num_batched_tokens, gpu_memory_utilization, num_blocks, use_cuda_graphs, seed).
        With ``model_config`` and ``random_weights`` the weights are drawn on the device and no
        folder is read."""
        t0 = time.time()
        self.cfg = EngineConfig(model=model, **engine_options)
        self.runner = ModelRunner(self.cfg, model_config=model_config,
                                  random_weights=random_weights, verbose=verbose)
        self.tokenizer = load_tokenizer(model) if model else None
        self.stop_ids = _stop_ids(model, self.tokenizer)
        self.scheduler = Scheduler(self.runner.manager, self.cfg.max_num_seqs,
                                   self.cfg.max_num_batched_tokens)
        self.sampler = Sampler(self.cfg.seed, self.runner.device, self.cfg.max_num_seqs)
        if self.cfg.use_cuda_graphs:
            self.runner.capture_decode_graphs()
        self.requests: dict = {}
        self.detok: dict = {}
        self.num_prompt_tokens_run = 0
        self.num_generated_tokens = 0
        self.num_steps = 0
        self._tokens_host = torch.empty(self.cfg.max_num_seqs, dtype=torch.int32).pin_memory()
        self.async_scheduling = async_scheduling
        self._token_bufs = [torch.empty(self.cfg.max_num_seqs, dtype=torch.int32).pin_memory() for _ in range(2)]
        # the slots of a step's wanted rows, when not every request of the step wants logits: staged
        # in pinned memory like the tokens, and reused only after that step's tokens have arrived
        self._slot_bufs = [torch.empty(self.cfg.max_num_seqs, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._slot_devs = [torch.empty(self.cfg.max_num_seqs, dtype=torch.int32, device=self.runner.device)
                           for _ in range(2)]
        self._flip = 0
        self._next = None          # _Packed: scheduled and packed, not launched
        self._in_flight = None     # _Sampled: sampled on the device, not read back
        self._spare_slot = self.cfg.max_num_seqs
        if verbose:
            print(f"[tinyserve_b200] engine ready in {time.time() - t0:.1f}s", flush=True)

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt, params: SamplingParams, request_id: Optional[str] = None) -> str:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs tokenizer files in the model folder; "
                                 "pass token ids instead")
            ids = self.tokenizer.encode(prompt)
        else:
            ids = [int(t) for t in prompt]
        if not 0 < len(ids) < self.cfg.max_model_len:
            raise ValueError(f"prompt of {len(ids)} tokens: must be 1..max_model_len-1 "
                             f"({self.cfg.max_model_len - 1})")
        vocab = self.runner.model.vocab_size
        if any(t < 0 or t >= vocab for t in ids):
            raise ValueError(f"prompt holds a token id outside [0, {vocab})")
        capacity = (self.runner.num_pages - 1) * self.runner.page_size
        if len(ids) + 1 > capacity:
            raise ValueError(f"prompt of {len(ids)} tokens does not fit the cache of {capacity} tokens")
        rid = request_id or uuid.uuid4().hex
        if rid in self.requests:
            raise ValueError(f"request id {rid!r} is in use")
        self.requests[rid] = req = Request(rid, ids, params)
        self.scheduler.add(req)
        self.detok[rid] = Detokenizer(self.tokenizer)
        return rid

    def abort(self, request_id: str) -> None:
        """Stop a request and give its pages back (serve.py:2474-2479)."""
        req = self.requests.pop(request_id, None)
        if req is not None and not req.finished:
            self.scheduler.finish(req, "abort")
            self.detok.pop(request_id, None)
        # a packed step, or tokens on their way, that only concern ended requests are dropped
        if self._next is not None and all(s.req.finished for s in self._next.batch):
            self._next = None
        if self._in_flight is not None and all(r.request_id not in self.requests for _, r, _ in self._in_flight.rows):
            self._in_flight = None

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._next is not None or self._in_flight is not None

    # ------------------------------------------------------------------ one step
    def step(self) -> list:
        """One engine step; returns the outputs of the requests that got a token."""
        return self._step_pipelined() if self.async_scheduling else self._step_sync()

    def _plan(self):
        """Schedule the next step and pack it on the host.  Returns a _Packed or None."""
        batch = self.scheduler.schedule()
        if not batch:
            return None
        entries, wants = [], []
        for s in batch:
            req = s.req
            wanted = s.completes_prompt                    # the step reaches the request's last known token
            if not wanted:
                req.was_chunked_prefill = True
            if s.num_computed < req.prompt_len:
                self.num_prompt_tokens_run += min(s.num_new, req.prompt_len - s.num_computed)
            entries.append(StepEntry(req.request_id, req.token_ids[s.num_computed:s.num_computed + s.num_new],
                                     [s.num_new - 1] if wanted else []))
            wants.append(wanted)
        return _Packed(batch, wants, self.runner.prepare(entries))

    def _over_length(self, req: Request) -> bool:
        return len(req.output_ids) >= req.params.max_tokens or req.num_tokens >= self.cfg.max_model_len

    # The host runs one step ahead of the device, as tinyserve's engine does (serve.py:2509-2601): a
    # call launches the step that the call before packed, reads the tokens of the step before that,
    # samples the launched step on the device and packs the next one, with PENDING in the place of
    # every token that is still on the device.
    @torch.inference_mode()
    def _step_pipelined(self) -> list:
        packed, self._next = self._next, None
        logits = None
        if packed is not None:
            logits = self.runner.launch(packed.prepared)
            self.num_steps += 1
        outputs = self._collect(self._in_flight) if self._in_flight is not None else []
        self._in_flight = None
        outputs += [self._output(r) for r in self._take_dropped()]
        if logits is not None:
            self._in_flight = self._sample_on_device(packed, logits)
        self._next = self._plan()
        return outputs

    def _sample_on_device(self, packed, logits):
        """Sample the launched step; its tokens stay on the device (each at its request's state
        slot, where the next step's embedding lookup finds it) and start their way to the host."""
        rows = [s.req for s, wanted in zip(packed.batch, packed.wants) if wanted]       # one per row of logits
        n = len(rows)
        if n == len(packed.batch):
            slots = self.runner.state_slots_on_device(n)
        else:
            manager = self.runner.manager
            staged = self._slot_bufs[self._flip]
            staged[:n] = torch.tensor([manager.slot(r.request_id) if manager.is_live(r.request_id)
                                       else self._spare_slot for r in rows], dtype=torch.int32)
            slots = self._slot_devs[self._flip][:n]
            slots.copy_(staged[:n], non_blocking=True)
        raw = logits.clone() if any(r.params.return_logprobs for r in rows) else None
        tokens_dev = self.sampler(logits, rows, slot_tokens=self.runner.slot_tokens, slots=slots)
        host = self._token_bufs[self._flip]
        self._flip ^= 1
        host[:n].copy_(tokens_dev, non_blocking=True)
        arrived = torch.cuda.Event()
        arrived.record()
        waiting_for = []
        for row, req in enumerate(rows):
            if req.finished:
                continue                   # ended (stop string, abort) after this step was packed
            forced = req.params.forced_token_ids
            req.token_ids.append(int(forced[len(req.output_ids)]) if forced is not None else PENDING)
            self.num_generated_tokens += 1
            if self._over_length(req):
                # its last token is on its way; nothing more is scheduled for it
                self.scheduler.finish(req, "length")
            waiting_for.append((row, req, len(req.token_ids) - 1))
        return _Sampled(waiting_for, host, arrived, raw)

    def _collect(self, flight) -> list:
        """The tokens of a sampled step have arrived (or are waited for): fill them in, look for
        stop tokens, make the outputs."""
        flight.arrived.synchronize()
        self.runner.raise_on_device_error()
        tokens = flight.host.tolist()
        outputs = []
        for row, req, at in flight.rows:
            if req.request_id not in self.requests:
                continue               # aborted meanwhile
            if req.token_ids[at] == PENDING:
                req.token_ids[at] = tokens[row]
            tok = req.token_ids[at]
            if req.params.return_logprobs:
                req.logprobs.append(flight.raw[row].log_softmax(-1).cpu())
            if tok in self.stop_ids and not req.params.ignore_eos:
                if req.finished:
                    req.finish_reason = "stop"
                else:
                    self.scheduler.finish(req, "stop")
            outputs.append(self._output(req))
        return outputs

    # ------------------------------------------------------------------ one step at a time
    @torch.inference_mode()
    def _step_sync(self) -> list:
        outputs = []
        packed = self._plan()
        outputs += [self._output(r) for r in self._take_dropped()]
        if packed is None:
            return outputs
        logits = self.runner.launch(packed.prepared)
        self.num_steps += 1
        rows = [s.req for s, wanted in zip(packed.batch, packed.wants) if wanted]
        if not rows:
            return outputs
        raw = logits.clone() if any(r.params.return_logprobs for r in rows) else None
        tokens_dev = self.sampler(logits, rows)
        n = len(rows)
        self._tokens_host[:n].copy_(tokens_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.runner.raise_on_device_error()
        tokens = self._tokens_host[:n].tolist()
        self.num_generated_tokens += n
        for row, req in enumerate(rows):
            forced = req.params.forced_token_ids
            tok = int(forced[len(req.output_ids)]) if forced is not None else tokens[row]
            req.token_ids.append(tok)
            if req.params.return_logprobs:
                req.logprobs.append(raw[row].log_softmax(-1).cpu())
            if tok in self.stop_ids and not req.params.ignore_eos:
                self.scheduler.finish(req, "stop")
            elif self._over_length(req):
                self.scheduler.finish(req, "length")
            outputs.append(self._output(req))
        return outputs

    def _take_dropped(self):
        dropped, self.scheduler.dropped = self.scheduler.dropped, []
        return dropped

    def _output(self, req: Request) -> Output:
        d = self.detok.get(req.request_id)
        text = delta = ""
        if d is not None and d.tok is not None:
            delta = d.update(req.output_ids, req.finished)
            text = d.text
            if req.params.stop:
                text, hit = apply_stop_strings(d.text, req.params.stop)
                if hit and not req.finished:
                    self.scheduler.finish(req, "stop")
                elif req.finished and not hit:
                    text = d.text
                delta, d.released = text[d.released:], len(text)
        out = Output(req.request_id, text, delta, req.output_ids, req.finished, req.finish_reason,
                     req.prompt_len, 0, req.logprobs if req.params.return_logprobs else None,
                     req.was_preempted, req.was_chunked_prefill)
        if req.finished:
            self.detok.pop(req.request_id, None)
            self.requests.pop(req.request_id, None)
        return out

    # ------------------------------------------------------------------ offline API
    def generate(self, prompts: list, params) -> list:
        """Add every prompt, step until all are done; outputs in request order."""
        params = params if isinstance(params, list) else [params] * len(prompts)
        rids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        done: dict = {}
        while self.has_work():
            for o in self.step():
                if o.finished:
                    done[o.request_id] = o
        return [done[r] for r in rids]

    def stats(self) -> dict:
        """The figures of tinyserve's log line (serve.py:2494-2507)."""
        return {"prompt_tokens_run": self.num_prompt_tokens_run,
                "generated_tokens": self.num_generated_tokens, "steps": self.num_steps,
                "running": len(self.scheduler.running), "waiting": len(self.scheduler.waiting),
                "kv_cache_usage": self.runner.manager.usage()}
