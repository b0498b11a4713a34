"""spyinfer_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

    from spyinfer_b200 import LLMEngine, SamplingParams
    engine = LLMEngine("/path/to/model", dtype="bfloat16")
    outputs = engine.generate([[1, 2, 3]], SamplingParams(max_new_tokens=8))
"""
from .config import EngineConfig, Qwen3Config, config_from_json, load_model_config
from .sampling import SamplingParams


def __getattr__(name):
    # the engine pulls in the CUDA side; configuration and weights work without it
    if name == "LLMEngine":
        from .engine.llm_engine import LLMEngine
        return LLMEngine
    raise AttributeError(name)


__all__ = ["LLMEngine", "SamplingParams", "EngineConfig", "Qwen3Config", "config_from_json", "load_model_config"]
