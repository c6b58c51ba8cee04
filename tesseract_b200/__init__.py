"""tesseract_b200: a single-GPU inference engine for NVIDIA B200 (sm_100a).

    from tesseract_b200 import LLM, SamplingParams
    outputs = LLM("/path/to/model").generate([[1, 2, 3]], SamplingParams(max_tokens=16, temperature=0.0))
"""

from .config import EngineConfig
from .sampling.params import SamplingParams

__all__ = ["LLM", "SamplingParams", "EngineConfig", "RequestOutput"]


def __getattr__(name):
    if name in ("LLM", "RequestOutput"):
        from .engine import llm

        return getattr(llm, name)
    raise AttributeError(name)
