"""Typed model configuration read from an architecture's own ``config.json`` keys.

``Qwen2Config`` carries every constant the Qwen2.5 dense decoder needs; nothing
in the parts or kernels hard-codes a size.  Key names, defaults and strictness
follow the reference reader (slipstream/models/hf_config.py:60-153): the five
required integers raise ``ConfigError`` when absent, ``head_dim`` defaults to
``hidden_size // num_attention_heads`` (:79-84), ``num_key_value_heads``
defaults to the head count (:86-87), ``attention_bias`` defaults to True for
``model_type`` qwen2 (:89-93), ``rms_norm_eps`` to 1e-6 (:138), ``rope_theta``
to 10000 and may sit inside ``rope_scaling`` (:103-105), ``hidden_act`` must be
``silu`` (:107-109), ``max_position_embeddings`` defaults to 4096 (:111-112),
token ids take the first element of a list and fall back to
``generation_config.json`` (:114-125).  ``torch_dtype`` names other than bfloat16 and float32
(the reference also takes float16, :248-262) are refused: this engine has two precisions.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any, ClassVar

from .reader import ConfigError, ConfigReader, load_json_object

read_json = load_json_object  # the name other modules import


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
        r = ConfigReader(data, behind=generation)
        model_type = r.text("model_type", "qwen2")
        hidden = r.integer("hidden_size")
        n_q = r.integer("num_attention_heads")
        head_dim = r.integer("head_dim", None)
        if head_dim is None:
            if n_q < 1 or hidden % n_q != 0:
                raise ConfigError(f"hidden_size {hidden} is not divisible by num_attention_heads {n_q}")
            head_dim = hidden // n_q

        rope = r.table("rope_scaling", "rope_parameters")
        rope_type = (rope.get("rope_type") or rope.get("type") or "default") if rope else "default"
        if rope_type != "default":
            raise ConfigError(f"rope type {rope_type!r} is not supported: this decoder uses the default "
                              "rotary frequencies only")
        theta = r.number("rope_theta", None)
        if theta is None:
            theta = ConfigReader(rope or {}, where="rope_scaling").number("rope_theta", 10000.0)

        if r.raw("use_sliding_window", False):
            # The reference reads none of the sliding-window keys and would run full attention where the
            # checkpoint asks for a window; refuse instead.
            raise ConfigError("use_sliding_window=true is not supported for Qwen2ForCausalLM "
                              "(its layers attend over all keys)")
        return cls(
            vocab_size=r.integer("vocab_size"),
            hidden_size=hidden,
            num_hidden_layers=r.integer("num_hidden_layers"),
            max_position_embeddings=r.integer("max_position_embeddings", 4096),
            torch_dtype=r.precision("torch_dtype", "dtype"),
            eos_token_id=r.token_id("eos_token_id"),
            bos_token_id=r.token_id("bos_token_id"),
            pad_token_id=r.token_id("pad_token_id"),
            intermediate_size=r.integer("intermediate_size"),
            num_attention_heads=n_q,
            num_key_value_heads=r.integer("num_key_value_heads", n_q),
            head_dim=head_dim,
            rms_norm_eps=r.number("rms_norm_eps", 1e-6),
            rope_theta=theta,
            tie_word_embeddings=r.flag("tie_word_embeddings", False),
            attention_bias=r.flag("attention_bias", model_type in ("qwen2", "qwen")),
            mlp_bias=r.flag("mlp_bias", False),
            hidden_act=r.text("hidden_act", "silu"),
            model_type=model_type,
            extra=r.leftover(also_known=("architectures",)),
        )

    def to_dict(self) -> dict[str, Any]:
        out = super().to_dict()
        extra = out.pop("extra")
        for key in ("eos_token_id", "bos_token_id", "pad_token_id"):
            if out[key] is None:
                del out[key]
        out.update({k: v for k, v in extra.items() if k not in out})
        return out
