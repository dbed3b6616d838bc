"""Engine options.  Names and meanings follow tinyserve's ``Config`` dataclass and
its command line (serve.py:76-122, 3098-3142) where it has them; ``dtype``,
``num_blocks`` and ``block_size`` are this engine's own."""
from __future__ import annotations

from dataclasses import dataclass


#: what ``check_indices`` is when an engine is configured without saying (tests switch it on)
CHECK_INDICES_DEFAULT = False

DTYPE_NAMES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32"}


@dataclass
class EngineConfig:
    model: str                          # model folder (config.json + *.safetensors)
    dtype: str = "bfloat16"             # "bfloat16" (serving) or "float32" (true 32-bit)
    max_model_len: int = 4096           # prompt + output cap; also the rotary table length
    block_size: int = 0                 # tokens per cache page (a power of two); 0 = chosen from max_model_len
    max_num_seqs: int = 128             # most requests in one step
    max_num_batched_tokens: int = 2048  # token budget of one step
    gpu_memory_utilization: float = 0.85
    num_blocks: int = 0                 # pages per cache group; 0 = size from memory
    use_cuda_graphs: bool = True        # replay captured decode steps
    seed: int = 0
    device: str = "cuda:0"
    # debug pass: check every index buffer of every step on the host before it is uploaded, and
    # again on the device before the kernels run (the stand-in for a memory checker)
    check_indices: bool = None

    def __post_init__(self):
        if self.check_indices is None:
            self.check_indices = CHECK_INDICES_DEFAULT
        if self.dtype not in DTYPE_NAMES:
            raise ValueError(f"dtype must be one of {sorted(DTYPE_NAMES)}, got {self.dtype!r}")
        self.dtype = DTYPE_NAMES[self.dtype]
        if self.block_size == 0:
            # tinyserve's pages hold 16 tokens (serve.py:114-115).  Pages of 64 let the decode kernel
            # fetch whole pages by TMA and the prefill kernel walk fewer of them (measured on B200 at
            # Qwen3-8B shapes: +3 % decode at batch 64, +4 % prefill); short contexts keep the small pages
            self.block_size = 64 if self.max_model_len >= 2048 else 16
        if self.block_size <= 0 or self.block_size & (self.block_size - 1):
            raise ValueError("block_size must be a power of two")
        if self.max_model_len <= 1:
            raise ValueError("max_model_len must exceed 1")
        if self.max_num_seqs <= 0 or self.max_num_batched_tokens <= 0:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be positive")
