"""cppvllm_b200: a small, whole inference engine for Qwen3 dense decoders on one NVIDIA B200 (sm_100a).

    from cppvllm_b200 import LLM, SamplingParams
    llm = LLM("/path/to/model", dtype="bfloat16")
    outs = llm.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=16))

Importing the package needs no GPU; building an engine does.
"""
from .config.engine_config import EngineConfig
from .sampling.params import SamplingParams

__all__ = ["EngineConfig", "SamplingParams", "LLM", "LLMEngine", "GenerationOutput"]


def __getattr__(name):
    if name in ("LLM", "LLMEngine", "GenerationOutput", "StepInfo", "EngineStats"):
        from .engine import llm_engine
        return getattr(llm_engine, name)
    raise AttributeError(f"module 'cppvllm_b200' has no attribute '{name}'")
