"""One registry from an architecture's name to its configuration class and model builder.

``config.json``'s ``architectures[0]`` picks the entry; a folder without that key
falls back on ``model_type`` (the reference dispatches on ``model_type`` alone,
slipstream/models/loader.py:50-55).  Another architecture is added with
``register_architecture(name, ConfigClass, builder, model_types=(...))``.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from slipstream_b200.config.model_config import ConfigError, ModelConfigBase, Qwen2Config, read_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build: Callable[[Any], Any]
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build: Callable[[Any], Any],
                          model_types: tuple[str, ...] = ()) -> None:
    if name in _ARCHITECTURES:
        raise KeyError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_class, build, tuple(model_types))


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(data: dict[str, Any]) -> Architecture:
    names = data.get("architectures")
    if isinstance(names, list) and names:
        name = names[0]
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
        raise ConfigError(f"unsupported architecture {name!r} (registered: {', '.join(architectures())})")
    model_type = data.get("model_type")
    for arch in _ARCHITECTURES.values():
        if model_type in arch.model_types:
            return arch
    raise ConfigError(f"unsupported model_type: {model_type!r} (registered architectures: "
                      f"{', '.join(architectures())})")


def load_config(folder: str | Path) -> tuple[Architecture, ModelConfigBase]:
    """Read ``config.json`` (and ``generation_config.json`` for token ids) of a model folder."""
    folder = Path(folder)
    cfg_path = folder / "config.json" if folder.is_dir() else folder
    if not cfg_path.is_file():
        raise FileNotFoundError(f"missing config.json at {cfg_path}")
    data = read_json(cfg_path)
    gen_path = cfg_path.parent / "generation_config.json"
    generation = read_json(gen_path) if gen_path.is_file() else None
    arch = resolve_architecture(data)
    return arch, arch.config_class.from_dict(data, generation)


def _register_builtin() -> None:
    from slipstream_b200.models.qwen2 import build_qwen2

    register_architecture("Qwen2ForCausalLM", Qwen2Config, build_qwen2, model_types=("qwen2", "qwen"))


_register_builtin()
