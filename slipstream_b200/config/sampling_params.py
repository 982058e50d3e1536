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
        # (field, admissible?, what to say): the ranges of slipstream/core/sampling_params.py:30-44
        rules = (
            ("max_tokens", self.max_tokens >= 1, "at least 1"),
            ("temperature", self.temperature >= 0.0, "zero (greedy) or positive"),
            ("top_k", self.top_k == -1 or self.top_k >= 1, "-1 (off) or at least 1"),
            ("top_p", 0.0 < self.top_p <= 1.0, "above 0 and at most 1"),
            ("min_p", 0.0 <= self.min_p <= 1.0, "between 0 and 1"),
            ("repetition_penalty", self.repetition_penalty > 0.0, "positive"),
            ("n", self.n == 1, "1: several samples of one prompt are not implemented"),
        )
        for name, ok, wanted in rules:
            if not ok:
                raise ValueError(f"{name}={getattr(self, name)!r}: must be {wanted}")
        object.__setattr__(self, "stop_token_ids", tuple(int(t) for t in self.stop_token_ids))
        object.__setattr__(self, "stop_strings", tuple(self.stop_strings))

    @property
    def is_greedy(self) -> bool:
        """Greedy when the temperature is zero or only the best token survives top-k
        (slipstream/core/sampling_params.py:46-48)."""
        return self.temperature == 0.0 or self.top_k == 1
