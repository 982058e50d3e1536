"""Engine-level options: dtype, cache pool, scheduler budgets.

Field names follow the reference's ``ModelConfig`` / ``CacheConfig`` /
``SchedulerConfig`` / ``EngineConfig`` (slipstream/core/config.py:25-134) where
it has them.  Differences: ``block_size`` may be any positive integer (the
reference allows 8, 16, 32 only, :71-72); ``max_model_len`` defaults to the
checkpoint's ``max_position_embeddings`` instead of a silent 4096 cap;
preemption is by recompute only, so there is no swap space.
"""

from __future__ import annotations

from dataclasses import dataclass, field

DEFAULT_BLOCK_SIZE = 16  # slipstream/core/types.py:23


@dataclass
class ModelOptions:
    model_id: str
    dtype: str | None = None  # bfloat16 | float32; None takes config.json's torch_dtype
    max_model_len: int | None = None  # None takes max_position_embeddings
    load_format: str = "safetensors"  # safetensors | random (weights drawn on the device)

    def __post_init__(self) -> None:
        if self.dtype is not None and self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"unsupported dtype: {self.dtype} (bfloat16 or float32)")
        if self.max_model_len is not None and self.max_model_len < 1:
            raise ValueError("max_model_len must be >= 1")
        if self.load_format not in ("safetensors", "random"):
            raise ValueError(f"unknown load_format: {self.load_format}")


@dataclass
class CacheConfig:
    block_size: int = DEFAULT_BLOCK_SIZE
    gpu_memory_utilization: float = 0.90
    num_gpu_blocks: int | None = None  # None: sized from free device memory

    def __post_init__(self) -> None:
        if self.block_size < 1:
            raise ValueError("block_size must be >= 1")
        if not (0.0 < self.gpu_memory_utilization <= 1.0):
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
        if self.num_gpu_blocks is not None and self.num_gpu_blocks < 1:
            raise ValueError("num_gpu_blocks must be >= 1")


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    enable_chunked_prefill: bool = True
    prefill_chunk_size: int = 256
    policy: str = "fcfs"

    def __post_init__(self) -> None:
        if self.policy != "fcfs":
            raise ValueError(f"unknown scheduling policy: {self.policy} (only fcfs is built)")
        if self.max_num_seqs < 1:
            raise ValueError("max_num_seqs must be >= 1")
        if self.max_num_batched_tokens < 1:
            raise ValueError("max_num_batched_tokens must be >= 1")
        if self.prefill_chunk_size < 1:
            raise ValueError("prefill_chunk_size must be >= 1")


@dataclass
class EngineConfig:
    model: ModelOptions
    cache: CacheConfig = field(default_factory=CacheConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    seed: int = 0
    use_cuda_graphs: bool = True

    @classmethod
    def for_model(cls, model_id: str, *, dtype: str | None = None,
                  max_model_len: int | None = None, load_format: str = "safetensors",
                  cache: CacheConfig | None = None, scheduler: SchedulerConfig | None = None,
                  seed: int = 0, use_cuda_graphs: bool = True) -> "EngineConfig":
        return cls(
            model=ModelOptions(model_id=model_id, dtype=dtype, max_model_len=max_model_len,
                               load_format=load_format),
            cache=cache if cache is not None else CacheConfig(),
            scheduler=scheduler if scheduler is not None else SchedulerConfig(),
            seed=seed,
            use_cuda_graphs=use_cuda_graphs,
        )
