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
    """Decides, step by step, which requests run and with how many tokens.

    ``running`` holds the requests that own pages and a state slot, oldest first; ``waiting``
    those that do not, in arrival order, preempted ones in front.  A step's grants are built in
    running order: first the running requests take what they owe from the token budget (pushing
    out the newest ones when the cache manager has no pages for them), then, if nobody was
    pushed out, the head of the waiting queue is let in for as long as budget, ``max_num_seqs``,
    state slots and pages last."""

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

    # ------------------------------------------------------------------ one step
    def schedule(self) -> list:
        grants: list = []                      # (request, tokens), in running order
        left = self.max_num_batched_tokens
        pushed_out = False
        at = 0
        while at < len(self.running) and left > 0:
            req = self.running[at]
            owed = min(req.num_tokens - req.num_computed_tokens, left)
            kept, evicted = self._room_for(req, owed)
            pushed_out = pushed_out or evicted
            if not kept:
                break                          # the request itself had to go: nobody after it runs
            grants.append((req, owed))
            left -= owed
            at += 1
        if not pushed_out:
            left = self._admit(grants, left)
        batch = []
        for req, n in grants:
            batch.append(ScheduledRequest(req, req.num_computed_tokens, n))
            req.num_computed_tokens += n       # counted before the device has run them
        return batch

    def _room_for(self, req: Request, tokens: int) -> tuple:
        """Pages for ``tokens`` more tokens of a running request.  While the pools cannot give
        them, the newest running request loses its pages and goes back to the head of the queue
        (it is never older than ``req``).  Returns (req still runs, somebody was pushed out)."""
        mgr, evicted = self.manager, False
        while not mgr.allocate(req.request_id, tokens):
            newest = self.running.pop()
            if newest is req:
                if self.running:
                    self._back_to_queue(req)
                    return False, True
                # no other request holds a page and it still does not fit: it never will
                mgr.free(req.request_id)
                self._drop(req)
                return False, evicted
            self._back_to_queue(newest)
            evicted = True
        return True, evicted

    def _admit(self, grants: list, left: int) -> int:
        """Let waiting requests in, strictly in order: the head of the queue or nobody."""
        mgr = self.manager
        while self.waiting and left > 0 and len(self.running) < self.max_num_seqs and mgr.can_begin():
            req = self.waiting[0]
            first = min(req.num_tokens, left)
            mgr.begin(req.request_id)
            if not mgr.allocate(req.request_id, first):
                mgr.free(req.request_id)
                if self.running:
                    break                      # it waits for pages that running requests hold
                # the whole pool is free and the portion still does not fit
                self.waiting.popleft()
                self._drop(req)
                continue
            self.waiting.popleft()
            req.num_computed_tokens = 0
            self.running.append(req)
            grants.append((req, first))
            left -= first
        return left

    def _back_to_queue(self, req: Request) -> None:
        """Preemption by recomputation: pages and slot go back, the request starts over."""
        req.was_preempted = True
        self.manager.free(req.request_id)
        req.num_computed_tokens = 0
        self.waiting.appendleft(req)

    def _drop(self, req: Request) -> None:
        req.finished, req.finish_reason = True, "cache_full"
        self.dropped.append(req)

    def finish(self, req: Request, reason: str) -> None:
        """End a request and give back what it holds (serve.py:619-625)."""
        req.finished, req.finish_reason = True, reason
        if req in self.running:
            self.running.remove(req)
            self.manager.free(req.request_id)
        elif req in self.waiting:
            self.waiting.remove(req)
