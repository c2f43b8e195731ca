"""Registry of architectures and the reading of ``config.json``.

One table maps the name in ``config.json`` (``architectures[0]``, or ``model_type``)
to the typed configuration class and to the function that turns a configuration
into a model description.  An unknown name and a known name that cannot run give two
different errors, as in the reference (src/model/qwen_model.cpp:259-272, registry
table src/model/arch_registry.cpp:13-95).
"""
from __future__ import annotations

import json
import os
import inspect
from dataclasses import dataclass
from typing import Callable, Optional, Protocol, runtime_checkable


class ConfigError(ValueError):
    """A configuration that is missing a key, holds a bad value or names no known model."""


@runtime_checkable
class ArchitectureConfig(Protocol):
    """What the rest of the package asks of an architecture's typed configuration, whatever its own
    keys are.  The engine, the loader of random models and the command line use these and nothing
    else of a configuration; everything else is between the class and its own ``build_spec``.

        architecture              the registry name the configuration was read under
        max_position_embeddings   the longest context the model allows (caps the cache's reach)
        torch_dtype               "bfloat16" | "float32" | "float16": the type a written folder stores
        from_dict(d)              classmethod: config.json's object -> configuration; raises ConfigError
        to_dict()                 the config.json that reads back as this configuration

    and of the entry's ``build_spec(config, max_positions=None) -> ModelSpec``: the model as data,
    with position tables sized for ``max_positions`` (default: the configuration's own limit).
    """
    architecture: str
    max_position_embeddings: int
    torch_dtype: str

    def to_dict(self) -> dict: ...


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str                      # "Qwen3ForCausalLM"
    model_type: str                # "qwen3"
    supported: bool
    notes: str
    config_cls: Optional[type] = None       # a class that follows ArchitectureConfig
    build_spec: Optional[Callable] = None   # (config, max_positions=None) -> ModelSpec


_REGISTRY: dict[str, ArchitectureEntry] = {}


def register_architecture(entry: ArchitectureEntry, replace: bool = False) -> ArchitectureEntry:
    if entry.supported:
        # the protocol above, checked where an architecture enters the table
        cls = entry.config_cls
        lacks = [a for a in ("from_dict", "to_dict") if not callable(getattr(cls, a, None))]
        fields = getattr(cls, "__dataclass_fields__", None) or getattr(cls, "__annotations__", {})
        lacks += [a for a in ("architecture", "max_position_embeddings", "torch_dtype")
                  if a not in fields and not hasattr(cls, a)]
        if cls is None or lacks:
            raise ConfigError(f"architecture '{entry.name}': its configuration class lacks {', '.join(lacks) or 'everything'} "
                              f"(see ArchitectureConfig)")
        if not callable(entry.build_spec) or "max_positions" not in inspect.signature(entry.build_spec).parameters:
            raise ConfigError(f"architecture '{entry.name}': build_spec must be callable as "
                              f"build_spec(config, max_positions=None)")
    for key in (entry.name, entry.model_type):
        if key in _REGISTRY and _REGISTRY[key].name != entry.name and not replace:
            raise ConfigError(f"architecture key '{key}' is already registered")
    _REGISTRY[entry.name] = entry
    _REGISTRY[entry.model_type] = entry
    return entry


def known_architectures() -> list[ArchitectureEntry]:
    seen, out = set(), []
    for e in _REGISTRY.values():
        if e.name not in seen:
            seen.add(e.name)
            out.append(e)
    return out


def find_architecture(name: str) -> ArchitectureEntry:
    entry = _REGISTRY.get(name)
    if entry is None:
        known = ", ".join(sorted(e.name for e in known_architectures()))
        raise ConfigError(f"unknown architecture '{name}'; known architectures: {known}")
    if not entry.supported:
        raise ConfigError(f"architecture '{name}' is recognized but not runnable: {entry.notes}")
    return entry


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in '{model_dir}'")
    with open(path, "r", encoding="utf-8") as f:
        try:
            data = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from e
    if not isinstance(data, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return data


def architecture_name(data: dict) -> str:
    archs = data.get("architectures")
    if isinstance(archs, list) and archs:
        return str(archs[0])
    if "model_type" in data:
        return str(data["model_type"])
    raise ConfigError("config.json names no architecture (neither 'architectures' nor 'model_type')")


def config_from_dict(data: dict):
    """Typed configuration of whatever architecture ``data`` names."""
    entry = find_architecture(architecture_name(data))
    return entry.config_cls.from_dict(data)


def _stop_ids_of(value) -> list:
    if value is None:
        return []
    if isinstance(value, int):
        return [value]
    if isinstance(value, (list, tuple)) and all(isinstance(v, int) for v in value):
        return list(value)
    raise ConfigError(f"eos_token_id must be an integer or a list of integers, got {value!r}")


def config_from_dir(model_dir: str):
    """The folder's config.json, typed.  A generation_config.json beside it may name further
    stop tokens under ``eos_token_id``; they are added to config.json's own."""
    data = read_config_json(model_dir)
    path = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(path):
        with open(path, "r", encoding="utf-8") as f:
            try:
                extra = json.load(f)
            except json.JSONDecodeError as e:
                raise ConfigError(f"{path} is not valid JSON: {e}") from e
        if isinstance(extra, dict) and extra.get("eos_token_id") is not None:
            ids = _stop_ids_of(data.get("eos_token_id"))
            for v in _stop_ids_of(extra["eos_token_id"]):
                if v not in ids:
                    ids.append(v)
            data = dict(data, eos_token_id=ids)
    return config_from_dict(data)
