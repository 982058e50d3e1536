"""Typed model configuration read from an architecture's own ``config.json`` keys.

``Qwen2Config`` carries every constant the Qwen2.5 dense decoder needs; nothing
in the parts or kernels hard-codes a size.  Key names, defaults and strictness
follow the reference reader (slipstream/models/hf_config.py:60-153): the five
required integers raise ``KeyError`` when absent, ``head_dim`` defaults to
``hidden_size // num_attention_heads`` (:79-84), ``num_key_value_heads``
defaults to the head count (:86-87), ``attention_bias`` defaults to True for
``model_type`` qwen2 (:89-93), ``rms_norm_eps`` to 1e-6 (:138), ``rope_theta``
to 10000 and may sit inside ``rope_scaling`` (:103-105), ``hidden_act`` must be
``silu`` (:107-109), ``max_position_embeddings`` defaults to 4096 (:111-112),
token ids take the first element of a list and fall back to
``generation_config.json`` (:114-125).
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A ``config.json`` value is missing, mistyped or unsupported."""


def _as_int(value: object, name: str) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        if isinstance(value, float) and value.is_integer():
            return int(value)
        raise ConfigError(f"{name} must be an integer, got {type(value).__name__}: {value!r}")
    return int(value)


def _as_float(value: object, name: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"{name} must be a number, got {type(value).__name__}: {value!r}")
    return float(value)


def _as_bool(value: object, name: str) -> bool:
    if not isinstance(value, bool):
        raise ConfigError(f"{name} must be true or false, got {type(value).__name__}: {value!r}")
    return value


def _first_id(value: object) -> int | None:
    if value is None:
        return None
    if isinstance(value, bool):
        raise ConfigError("a token id must not be a boolean")
    if isinstance(value, int):
        return value
    if isinstance(value, list) and value:
        return _first_id(value[0])
    return None


_DTYPE_NAMES = {
    "bfloat16": "bfloat16",
    "bf16": "bfloat16",
    "float32": "float32",
    "fp32": "float32",
}


def read_json(path: Path) -> dict[str, Any]:
    with path.open(encoding="utf-8") as handle:
        data = json.load(handle)
    if not isinstance(data, dict):
        raise ConfigError(f"{path} is not a JSON object")
    return data


@dataclass(frozen=True)
class ModelConfigBase:
    """What every architecture's configuration exposes to the engine."""

    architecture: ClassVar[str] = ""

    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    max_position_embeddings: int = 4096
    torch_dtype: str = "bfloat16"
    eos_token_id: int | None = None
    bos_token_id: int | None = None
    pad_token_id: int | None = None

    def to_dict(self) -> dict[str, Any]:
        out = asdict(self)
        out["architectures"] = [self.architecture]
        return out


@dataclass(frozen=True)
class Qwen2Config(ModelConfigBase):
    """Qwen2.5 dense decoder: pre-norm RMSNorm, GQA attention with biased
    q/k/v, rotary positions, SwiGLU feed-forward, optional tied embeddings
    (slipstream/models/causal_lm.py:31-141)."""

    architecture: ClassVar[str] = "Qwen2ForCausalLM"

    intermediate_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    attention_bias: bool = True
    mlp_bias: bool = False
    hidden_act: str = "silu"
    model_type: str = "qwen2"
    extra: dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    def __post_init__(self) -> None:
        for name in ("vocab_size", "hidden_size", "num_hidden_layers", "intermediate_size",
                     "num_attention_heads", "num_key_value_heads", "head_dim",
                     "max_position_embeddings"):
            if getattr(self, name) < 1:
                raise ConfigError(f"{name} must be >= 1, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            # slipstream/models/layers/attention.py:114-115
            raise ConfigError(
                f"num_attention_heads ({self.num_attention_heads}) must be divisible by "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim must be even for rotary pairs, got {self.head_dim}")
        if self.hidden_act != "silu":
            raise ConfigError(f"unsupported hidden_act: {self.hidden_act}")
        if not self.rms_norm_eps > 0.0:
            raise ConfigError(f"rms_norm_eps must be > 0, got {self.rms_norm_eps}")
        if not self.rope_theta > 0.0:
            raise ConfigError(f"rope_theta must be > 0, got {self.rope_theta}")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"unsupported torch_dtype: {self.torch_dtype}")

    @classmethod
    def from_dict(cls, data: dict[str, Any], generation: dict[str, Any] | None = None) -> "Qwen2Config":
        def need(key: str) -> object:
            if key not in data or data[key] is None:
                raise ConfigError(f"config.json lacks the required key {key!r}")
            return data[key]

        model_type = data.get("model_type", "qwen2")
        if not isinstance(model_type, str):
            raise ConfigError(f"model_type must be a string, got {model_type!r}")
        hidden = _as_int(need("hidden_size"), "hidden_size")
        n_q = _as_int(need("num_attention_heads"), "num_attention_heads")
        if data.get("head_dim") is not None:
            head_dim = _as_int(data["head_dim"], "head_dim")
        else:
            if hidden % n_q != 0:
                raise ConfigError(
                    f"hidden_size {hidden} is not divisible by num_attention_heads {n_q}")
            head_dim = hidden // n_q
        n_kv = data.get("num_key_value_heads")
        n_kv = _as_int(n_kv, "num_key_value_heads") if n_kv is not None else n_q

        rope = data.get("rope_scaling")
        if rope is None:
            rope = data.get("rope_parameters")
        if rope is not None and not isinstance(rope, dict):
            raise ConfigError("rope_scaling / rope_parameters must be an object")
        rope_type = "default"
        if rope is not None:
            rope_type = rope.get("rope_type", rope.get("type", "default")) or "default"
        if rope_type != "default":
            raise ConfigError(
                f"rope type {rope_type!r} is not supported: this decoder uses the default "
                "rotary frequencies only")
        theta = data.get("rope_theta")
        if theta is None and rope is not None and "rope_theta" in rope:
            theta = rope["rope_theta"]

        if data.get("use_sliding_window"):
            # The reference reads none of the sliding-window keys and would run full
            # attention where the checkpoint asks for a window; refuse instead.
            raise ConfigError(
                "use_sliding_window=true is not supported for Qwen2ForCausalLM "
                "(its layers attend over all keys)")

        gen = generation or {}

        def token_id(key: str) -> int | None:
            found = _first_id(data.get(key))
            return found if found is not None else _first_id(gen.get(key))

        dtype_raw = data.get("torch_dtype", data.get("dtype"))
        dtype = _DTYPE_NAMES.get(dtype_raw, "bfloat16") if isinstance(dtype_raw, str) else "bfloat16"

        known = {
            "model_type", "hidden_size", "num_attention_heads", "num_hidden_layers", "vocab_size",
            "intermediate_size", "head_dim", "num_key_value_heads", "attention_bias", "mlp_bias",
            "rope_scaling", "rope_parameters", "rope_theta", "hidden_act",
            "max_position_embeddings", "eos_token_id", "bos_token_id", "pad_token_id",
            "torch_dtype", "dtype", "rms_norm_eps", "tie_word_embeddings", "architectures",
        }
        return cls(
            vocab_size=_as_int(need("vocab_size"), "vocab_size"),
            hidden_size=hidden,
            num_hidden_layers=_as_int(need("num_hidden_layers"), "num_hidden_layers"),
            max_position_embeddings=(
                _as_int(data["max_position_embeddings"], "max_position_embeddings")
                if data.get("max_position_embeddings") is not None else 4096),
            torch_dtype=dtype,
            eos_token_id=token_id("eos_token_id"),
            bos_token_id=token_id("bos_token_id"),
            pad_token_id=token_id("pad_token_id"),
            intermediate_size=_as_int(need("intermediate_size"), "intermediate_size"),
            num_attention_heads=n_q,
            num_key_value_heads=n_kv,
            head_dim=head_dim,
            rms_norm_eps=_as_float(data.get("rms_norm_eps", 1e-6), "rms_norm_eps"),
            rope_theta=_as_float(theta if theta is not None else 10000.0, "rope_theta"),
            tie_word_embeddings=(
                _as_bool(data["tie_word_embeddings"], "tie_word_embeddings")
                if data.get("tie_word_embeddings") is not None else False),
            attention_bias=(
                _as_bool(data["attention_bias"], "attention_bias")
                if data.get("attention_bias") is not None else model_type in ("qwen2", "qwen")),
            mlp_bias=(
                _as_bool(data["mlp_bias"], "mlp_bias")
                if data.get("mlp_bias") is not None else False),
            hidden_act=data.get("hidden_act") or "silu",
            model_type=model_type,
            extra={k: v for k, v in data.items() if k not in known},
        )

    def to_dict(self) -> dict[str, Any]:
        out = super().to_dict()
        extra = out.pop("extra")
        for key in ("eos_token_id", "bos_token_id", "pad_token_id"):
            if out[key] is None:
                del out[key]
        out.update({k: v for k, v in extra.items() if k not in out})
        return out
