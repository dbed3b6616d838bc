"""Continuous batching over the step function: who runs next, with how many tokens.

The rules are tinyserve's ``Scheduler.schedule`` (serve.py:475-617):
  * one token budget per step, shared by prompt portions and decoded tokens
    (serve.py:477-479);
  * running requests first, oldest first; each gets min(tokens it still owes, budget left):
    one token when it decodes, the rest of its prompt, or as much as fits, when it
    prefills (serve.py:491-499);
  * when pages run out, the newest running request is preempted: its pages and slot are
    given back, it starts from zero again at the front of the waiting queue, and the
    allocation is tried again (serve.py:505-555);
  * new requests are admitted in arrival order, only the head of the queue, only when
    nothing was preempted in this step, while budget and ``max_num_seqs`` allow
    (serve.py:567-602);
  * a prompt longer than the budget left is cut there and goes on in later steps
    (serve.py:499, 579).
Decided here, where tinyserve retries for ever (serve.py:544-550): a request that cannot
get pages although no other request holds any ends with reason "cache_full"."""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass


class Request:
    """A request as the scheduler sees it (serve.py:139-186)."""

    def __init__(self, request_id, prompt_ids, params):
        self.request_id = request_id
        self.prompt_len = len(prompt_ids)
        self.token_ids = list(prompt_ids)          # prompt + generated so far
        self.params = params
        self.num_computed_tokens = 0               # tokens whose keys and values are cached
        self.finished = False
        self.finish_reason = None
        self.was_preempted = False
        self.was_chunked_prefill = False
        self.logprobs = []

    @property
    def num_tokens(self):
        return len(self.token_ids)

    @property
    def output_ids(self):
        return self.token_ids[self.prompt_len:]


@dataclass
class ScheduledRequest:
    req: Request
    num_computed: int      # tokens cached before this step
    num_new: int           # tokens this step runs

    @property
    def completes_prompt(self):
        """True if this step runs the request's last known token, so its logits are wanted."""
        return self.num_computed + self.num_new >= self.req.num_tokens


class Scheduler:
    def __init__(self, manager, max_num_seqs: int, max_num_batched_tokens: int):
        self.manager = manager
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.waiting: deque = deque()
        self.running: list = []
        self.dropped: list = []     # requests ended by the scheduler itself ("cache_full")

    def add(self, req: Request) -> None:
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _preempt(self, victim: Request) -> None:
        victim.was_preempted = True
        self.manager.free(victim.request_id)
        victim.num_computed_tokens = 0
        self.waiting.appendleft(victim)

    def schedule(self) -> list:
        mgr = self.manager
        budget = self.max_num_batched_tokens
        plan: dict = {}
        preempted = False
        i = 0
        while i < len(self.running) and budget > 0:
            req = self.running[i]
            n = min(req.num_tokens - req.num_computed_tokens, budget)
            stop = False
            while not mgr.allocate(req.request_id, n):
                victim = self.running.pop()
                if victim is req and not self.running:
                    # nobody else holds pages: this request can never fit
                    mgr.free(req.request_id)
                    req.finished, req.finish_reason = True, "cache_full"
                    self.dropped.append(req)
                    stop = True
                    break
                self._preempt(victim)
                budget += plan.pop(victim.request_id, 0)
                preempted = True
                if victim is req:
                    stop = True
                    break
            if stop:
                break
            plan[req.request_id] = n
            budget -= n
            i += 1

        while (not preempted and self.waiting and budget > 0
               and len(self.running) < self.max_num_seqs and mgr.can_begin()):
            req = self.waiting[0]
            mgr.begin(req.request_id)
            n = min(req.num_tokens, budget)
            if not mgr.allocate(req.request_id, n):
                mgr.free(req.request_id)
                if not self.running:
                    # the pool is empty and the portion still does not fit
                    self.waiting.popleft()
                    req.finished, req.finish_reason = True, "cache_full"
                    self.dropped.append(req)
                    continue
                break
            self.waiting.popleft()
            req.num_computed_tokens = 0
            self.running.append(req)
            plan[req.request_id] = n
            budget -= n

        batch = []
        for req in self.running:
            n = plan.get(req.request_id)
            if n:
                batch.append(ScheduledRequest(req, req.num_computed_tokens, n))
                req.num_computed_tokens += n
        return batch

    def finish(self, req: Request, reason: str) -> None:
        """End a request and give back what it holds (serve.py:619-625)."""
        req.finished, req.finish_reason = True, reason
        if req in self.running:
            self.running.remove(req)
            self.manager.free(req.request_id)
        elif req in self.waiting:
            self.waiting.remove(req)
