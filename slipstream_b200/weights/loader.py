"""Weights from safetensors by tensor name.

Files are found as the reference finds them (slipstream/models/loader.py:105-126):
``model.safetensors.index.json`` -> the shards of its ``weight_map``; else
``model.safetensors``; else every ``*.safetensors``.  Tensors are matched against
the model's ``WeightSpec`` list.  All faults are gathered into ONE ``WeightError``
that lists missing tensors, unexpected tensors and wrong shapes (the reference
raises on the first wrong shape, lists missing ones, and only warns about
unexpected ones, :82-98).  Rotary buffers some exporters store are skipped (:26).

Kept dtypes: ``matrix`` tensors in the compute dtype; ``vector`` tensors too,
unless the file stores them in 32-bit, which is kept; ``index`` tensors as int32.
A tied tensor absent from the file aliases its source; present, it must be equal.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from slipstream_b200.parts.base import Runtime, WeightSpec

_SKIP_KEY_PARTS = ("inv_freq", "rotary_emb", "cos_cached", "sin_cached")


class WeightError(RuntimeError):
    """The checkpoint does not fit the model; the message lists every mismatch."""


def safetensor_files(folder: Path) -> list[Path]:
    index = folder / "model.safetensors.index.json"
    if index.is_file():
        weight_map = json.loads(index.read_text(encoding="utf-8")).get("weight_map")
        if not isinstance(weight_map, dict) or not weight_map:
            raise FileNotFoundError(f"empty weight_map in {index}")
        paths = [folder / name for name in sorted({str(v) for v in weight_map.values()})]
        for path in paths:
            if not path.is_file():
                raise FileNotFoundError(f"missing shard {path}")
        return paths
    single = folder / "model.safetensors"
    if single.is_file():
        return [single]
    shards = sorted(folder.glob("*.safetensors"))
    if shards:
        return shards
    raise FileNotFoundError(f"no safetensors weights under {folder}")


def _kept_dtype(spec: WeightSpec, stored: torch.dtype, runtime: Runtime) -> torch.dtype:
    if spec.kind == "index":
        return torch.int32
    if spec.kind == "vector" and stored == torch.float32:
        return torch.float32
    return runtime.dtype


def load_weights(folder: str | Path, specs: list[WeightSpec], runtime: Runtime) -> dict[str, torch.Tensor]:
    """Read every tensor the specs name onto the device; raise one error for all faults."""
    from safetensors import safe_open

    folder = Path(folder)
    by_name = {s.name: s for s in specs}
    out: dict[str, torch.Tensor] = {}
    unexpected: list[str] = []
    wrong_shape: list[str] = []
    non_finite: list[str] = []
    for shard in safetensor_files(folder):
        with safe_open(str(shard), framework="pt", device="cpu") as handle:
            for key in handle.keys():
                if any(part in key for part in _SKIP_KEY_PARTS):
                    continue
                spec = by_name.get(key)
                if spec is None:
                    unexpected.append(key)
                    continue
                shape = tuple(handle.get_slice(key).get_shape())
                if shape != tuple(spec.shape):
                    wrong_shape.append(f"{key}: file {shape} vs model {tuple(spec.shape)}")
                    continue
                tensor = handle.get_tensor(key)
                kept = tensor.to(device=runtime.device, dtype=_kept_dtype(spec, tensor.dtype, runtime))
                if kept.is_floating_point() and not torch.isfinite(kept).all():
                    non_finite.append(key)
                out[key] = kept.contiguous()
    missing: list[str] = []
    for spec in specs:
        if spec.name in out or any(w.startswith(spec.name + ":") for w in wrong_shape):
            continue
        if spec.alias_of is not None and spec.alias_of in out:
            out[spec.name] = out[spec.alias_of]
            continue
        missing.append(spec.name)
    tied_unequal = [s.name for s in specs
                    if s.alias_of is not None and s.name in out and s.alias_of in out
                    and out[s.name] is not out[s.alias_of] and not torch.equal(out[s.name], out[s.alias_of])]
    if missing or unexpected or wrong_shape or non_finite or tied_unequal:
        lines = [f"the weights under {folder} do not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): {', '.join(sorted(missing))}")
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): {', '.join(sorted(unexpected))}")
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): {'; '.join(sorted(wrong_shape))}")
        if non_finite:
            lines.append(f"  non-finite values in: {', '.join(sorted(non_finite))}")
        if tied_unequal:
            lines.append(f"  tied tensors that differ from their source: {', '.join(sorted(tied_unequal))}")
        raise WeightError("\n".join(lines))
    return out
