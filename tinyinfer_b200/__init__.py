"""tinyinfer_b200: a small, whole inference engine for the Qwen3 dense decoder on one B200.

    from tinyinfer_b200 import LLM, SamplingParams
    llm = LLM("/path/to/model", max_num_seqs=8)
    out = llm.generate([[1, 2, 3]], SamplingParams(greedy=True, max_tokens=16))
"""
__version__ = "0.1.0"

from .config import EngineConfig
from .sampling import SamplingParams


def __getattr__(name):
    if name == "LLM":                      # imported late: it pulls in torch and the engine
        from .engine.llm import LLM
        return LLM
    raise AttributeError(name)


__all__ = ["LLM", "SamplingParams", "EngineConfig"]
