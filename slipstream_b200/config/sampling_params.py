"""Per-request sampling options, with the reference's names, defaults and checks
(slipstream/core/sampling_params.py:8-48).

``n`` above 1 is rejected: the reference declares it but never forks a sequence.
``stop_strings`` need a tokenizer in the model folder.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class SamplingParams:
    max_tokens: int = 16
    temperature: float = 1.0
    top_k: int = -1  # -1 disables
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    stop_token_ids: tuple[int, ...] = ()
    stop_strings: tuple[str, ...] = ()
    ignore_eos: bool = False
    seed: int | None = None
    n: int = 1
    extra: dict[str, object] = field(default_factory=dict, hash=False, compare=False)

    def __post_init__(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        if self.temperature < 0.0:
            raise ValueError("temperature must be >= 0")
        if self.top_k == 0 or self.top_k < -1:
            raise ValueError("top_k must be -1 or >= 1")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError("min_p must be in [0, 1]")
        if self.repetition_penalty <= 0.0:
            raise ValueError("repetition_penalty must be > 0")
        if self.n != 1:
            raise ValueError("n must be 1: parallel sampling of one prompt is not implemented")
        object.__setattr__(self, "stop_token_ids", tuple(int(t) for t in self.stop_token_ids))
        object.__setattr__(self, "stop_strings", tuple(self.stop_strings))

    @property
    def is_greedy(self) -> bool:
        """Greedy when the temperature is zero or only the best token survives top-k
        (slipstream/core/sampling_params.py:46-48)."""
        return self.temperature == 0.0 or self.top_k == 1
