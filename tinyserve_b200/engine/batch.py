"""What one step is given and what the parts see of it."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class StepEntry:
    """A request's next tokens.  ``want``: places among ``tokens`` whose logits are asked."""

    rid: object
    tokens: list
    want: list = field(default_factory=list)


@dataclass
class GroupView:
    """One cache group as this step sees it."""

    page_size: int
    max_blocks: int
    slot_mapping: torch.Tensor      # int32 [T]: page * page_size + slot of each new token, -1 = none
    block_table: torch.Tensor       # int32 [B, max_blocks]
    num_pages: int = 0              # pages of the group's pool (the null page included)


class StepContext:
    """Device views of one step's batch plus the cache; passed to every part.

    token_ids, positions: int32 [T].  cu_q: int32 [B + 1], prefix sums of the requests'
    token counts.  kv_lens: int32 [B], tokens each request holds after this step.
    state_slots: int32 [B].  fresh: int32 [B], 1 if the request's first token is in this
    step (its state starts at zero).  logit_rows: int32 [W] rows of the batch whose logits
    are wanted.  Host copies of the small arrays are in ``host``."""

    def __init__(self):
        self.num_tokens = 0
        self.num_requests = 0
        self.max_q_len = 0
        self.max_kv_len = 0
        self.decode_only = False
        self.num_logit_rows = 0
        self.token_ids = self.positions = self.cu_q = self.kv_lens = None
        self.state_slots = self.fresh = self.logit_rows = None
        self.groups: list = []
        self.device_cache = None
        self.host: dict = {}
        self.dtype = None
        self.workspace = None
        self.slot_tokens = None      # int32 [slots + 1]: last sampled token of every state slot
        self.tile_cache: dict = {}   # attention work lists of this step, by queries per block

    def cache(self, index: int):
        return self.device_cache.entries[index]

    def group(self, index: int) -> GroupView:
        return self.groups[index]

    def state(self, index: int) -> torch.Tensor:
        return self.device_cache.states[index]
