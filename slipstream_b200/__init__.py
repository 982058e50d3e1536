"""slipstream_b200: a small, whole inference engine for the Qwen2.5 dense decoder on one B200.

Model folder (config.json + safetensors) -> tokens: typed configuration and an
architecture registry, a safetensors loader with a random-weights mode, layers put
together from parts, a paged key/value cache with per-request block tables and
state slots, one step function over mixed batches, a continuous-batching
scheduler, sampling, a CLI, a Python entry point and a trace-replay tool, all on
hand-written sm_100a CUDA kernels.
"""

__version__ = "0.1.0"

from .config.engine_config import CacheConfig, EngineConfig, ModelConfig, ModelOptions, ParallelConfig, SchedulerConfig
from .config.sampling_params import SamplingParams

__all__ = ["CacheConfig", "EngineConfig", "ModelConfig", "ModelOptions", "ParallelConfig", "SchedulerConfig", "SamplingParams",
           "LLM", "LLMEngine", "Request"]


def __getattr__(name: str):
    if name in ("LLM", "LLMEngine", "Request", "RequestOutput"):
        from .engine import llm_engine

        return getattr(llm_engine, name)
    raise AttributeError(name)
