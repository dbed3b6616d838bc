"""Per-request sampling options; names, defaults and meanings are tinyserve's
(serve.py:124-137).  ``seed`` is this engine's: it selects the request's noise stream."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


@dataclass
class SamplingParams:
    temperature: float = 1.0          # 0 means greedy decoding
    top_p: float = 1.0
    top_k: int = -1                   # -1 means off
    max_tokens: int = 64
    repetition_penalty: float = 1.1   # > 1 makes recent tokens less likely, 1.0 = off
    repeat_last_n: int = 64           # recent tokens the penalty looks at, 0 = off, -1 = all
    ignore_eos: bool = False
    stop: Optional[list] = None       # strings that end the generation
    forced_token_ids: Optional[list] = None   # teacher forcing, for tests
    return_logprobs: bool = False
    seed: Optional[int] = None        # noise stream of this request (default: from its id)

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0 < self.top_p <= 1:
            raise ValueError("top_p must lie in (0, 1]")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if self.repetition_penalty <= 0:
            raise ValueError("repetition_penalty must be positive")
