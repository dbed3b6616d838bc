"""tinyserve_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a).

    from tinyserve_b200 import LLM, SamplingParams
    out = LLM("model_dir").generate([[1, 2, 3]], SamplingParams(temperature=0, max_tokens=8))
"""
__version__ = "0.1.0"

from .config import EngineConfig, Qwen3Config, load_model_config, register_architecture  # noqa: F401
from .sampling import SamplingParams  # noqa: F401


def __getattr__(name):
    if name in ("LLM", "Output"):
        from .engine import llm
        return getattr(llm, name)
    raise AttributeError(name)
