"""Random-weights mode: draw every tensor of a model from a seed.

``write_random_model`` writes a model folder (``config.json`` and
``model.safetensors``) from a configuration and a seed, so that any reader of the
format, this engine's loader included, sees the same weights.  Each tensor is
drawn on the CPU from a generator seeded by (seed, tensor name): the result
depends neither on the order of drawing nor on the device.  Matrices, embeddings
and biases are N(0, std); norm weights are 1 + N(0, std); the standard deviations
come from the parts' ``WeightSpec.init``.

``random_weights_on_device`` draws the same kinds of tensors directly on the
device for benchmarks of large shapes (different values from the CPU draw).
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from slipstream_b200.parts.base import Runtime, WeightSpec

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def draw_tensor(spec: WeightSpec, seed: int, dtype: torch.dtype) -> torch.Tensor:
    gen = torch.Generator(device="cpu")
    gen.manual_seed(_tensor_seed(seed, spec.name))
    kind, std = spec.init
    if spec.kind == "index":
        return torch.zeros(spec.shape, dtype=torch.int32)
    values = torch.randn(spec.shape, generator=gen, dtype=torch.float32) * std
    if kind == "one_plus_normal":
        values += 1.0
    elif kind != "normal":
        raise ValueError(f"unknown init {kind!r} for {spec.name}")
    return values.to(dtype)


def write_random_model(config, out_dir: str | Path, seed: int = 0, dtype: str | None = None) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed model configuration
    of a registered architecture) with weights drawn from ``seed``.  Tied tensors are not stored."""
    from safetensors.torch import save_file

    from slipstream_b200.registry import resolve_architecture

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    data = config.to_dict()
    if dtype is not None:
        data["torch_dtype"] = dtype
    arch = resolve_architecture(data)
    model = arch.build(config)
    torch_dtype = _DTYPES[data.get("torch_dtype", "bfloat16")]
    tensors = {}
    for spec in model.weight_specs():
        if spec.alias_of is not None:
            continue
        tensors[spec.name] = draw_tensor(spec, seed, torch_dtype).contiguous()
    (out / "config.json").write_text(json.dumps(data, indent=2) + "\n", encoding="utf-8")
    save_file(tensors, str(out / "model.safetensors"), metadata={"format": "pt"})
    return out


def random_weights_on_device(specs: list[WeightSpec], runtime: Runtime, seed: int = 0) -> dict[str, torch.Tensor]:
    gen = torch.Generator(device=runtime.device)
    gen.manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for spec in specs:
        if spec.alias_of is not None:
            continue
        if spec.kind == "index":
            out[spec.name] = torch.zeros(spec.shape, dtype=torch.int32, device=runtime.device)
            continue
        kind, std = spec.init
        t = torch.empty(spec.shape, dtype=runtime.dtype, device=runtime.device)
        t.normal_(0.0, std, generator=gen)
        if kind == "one_plus_normal":
            t += 1.0
        out[spec.name] = t
    for spec in specs:
        if spec.alias_of is not None:
            out[spec.name] = out[spec.alias_of]
    return out
