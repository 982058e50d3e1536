"""Engine-level options: dtype, cache pool, scheduler budgets.

Field names follow the reference's ``ModelConfig`` / ``CacheConfig`` /
``SchedulerConfig`` / ``EngineConfig`` (slipstream/core/config.py:25-134) where
it has them.  Differences: ``block_size`` may be any positive integer (the
reference allows 8, 16, 32 only, :71-72); ``max_model_len`` defaults to the
checkpoint's ``max_position_embeddings`` instead of a silent 4096 cap;
preemption is by recompute only, so no swap space is allocated.  Fields of the
reference that belong to parts that are not built here (prefix caching, the
unpaged path, swap space, the Horizon policy's knobs, tensor parallelism) are
kept, so that a configuration written for the reference still constructs; a
value that asks for such a part is refused.
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


ModelConfig = ModelOptions  # the reference's name for it (slipstream/core/config.py:25-57)


@dataclass
class CacheConfig:
    block_size: int = DEFAULT_BLOCK_SIZE
    gpu_memory_utilization: float = 0.90
    swap_space_bytes: int = 4 * 1024**3  # not used: a preempted request is recomputed
    enable_prefix_caching: bool = False  # sharing of prompt prefixes is not built
    enable_paging: bool = True  # the cache is always paged
    num_gpu_blocks: int | None = None  # None: sized from free device memory
    num_cpu_blocks: int | None = None  # not used (no swap space)

    def __post_init__(self) -> None:
        if self.block_size < 1:
            raise ValueError("block_size must be >= 1")
        if self.enable_prefix_caching:
            raise ValueError("enable_prefix_caching=True: prefix caching is not built in this engine")
        if not self.enable_paging:
            raise ValueError("enable_paging=False: this engine has no unpaged cache")
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
    max_wait_ms: float = 30_000.0  # the three below steer the reference's other policies; fcfs reads none
    safety_factor: float = 0.95
    starvation_guard_ms: float = 5_000.0

    def __post_init__(self) -> None:
        if self.policy != "fcfs":
            raise ValueError(f"unknown scheduling policy: {self.policy} (only fcfs is built)")
        if not (0.0 < self.safety_factor <= 1.0):
            raise ValueError("safety_factor must be in (0, 1]")
        if self.max_num_seqs < 1:
            raise ValueError("max_num_seqs must be >= 1")
        if self.max_num_batched_tokens < 1:
            raise ValueError("max_num_batched_tokens must be >= 1")
        if self.prefill_chunk_size < 1:
            raise ValueError("prefill_chunk_size must be >= 1")


@dataclass
class ParallelConfig:
    tensor_parallel_size: int = 1

    def __post_init__(self) -> None:
        if self.tensor_parallel_size != 1:
            raise ValueError("tensor_parallel_size must be 1: this engine runs on one GPU")


@dataclass
class EngineConfig:
    model: ModelOptions
    cache: CacheConfig = field(default_factory=CacheConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    seed: int = 0
    use_cuda_graphs: bool = True

    @classmethod
    def for_model(cls, model_id: str, *, dtype: str | None = None,
                  max_model_len: int | None = None, load_format: str = "safetensors",
                  cache: CacheConfig | None = None, scheduler: SchedulerConfig | None = None,
                  parallel: ParallelConfig | None = None, seed: int = 0,
                  use_cuda_graphs: bool = True) -> "EngineConfig":
        return cls(
            model=ModelOptions(model_id=model_id, dtype=dtype, max_model_len=max_model_len,
                               load_format=load_format),
            cache=cache if cache is not None else CacheConfig(),
            scheduler=scheduler if scheduler is not None else SchedulerConfig(),
            parallel=parallel if parallel is not None else ParallelConfig(),
            seed=seed,
            use_cuda_graphs=use_cuda_graphs,
        )
