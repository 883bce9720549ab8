"""One registry from an architecture's name to its configuration class and plan builder.

Reference: the reference dispatches on the ``model_type`` string with a ``match``
(src/engine.rs:663-669, src/main.rs:558-563; ``config::model_type`` src/config.rs:350-365) and
fails with ``unsupported model_type``.  Here both ``architectures[0]`` and ``model_type`` are
looked up in one table, and the error lists the known names.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Dict, Iterable, Optional

from .base import ConfigError, ModelConfig, read_config_json


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    #: (config, names of the checkpoint's tensors or None) -> ModelPlan
    build_plan: Callable
    #: config -> {tensor name: (shape, kind)} of a complete checkpoint, for random weights
    checkpoint_layout: Optional[Callable] = None


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(names: Iterable[str], config_class: type, build_plan: Callable,
                          checkpoint_layout: Optional[Callable] = None) -> None:
    """Registers an architecture under each of ``names`` (an ``architectures`` entry of
    config.json and/or a ``model_type``)."""
    if not issubclass(config_class, ModelConfig):
        raise TypeError("config_class must derive from ModelConfig")
    for n in names:
        _ARCHITECTURES[n] = Architecture(n, config_class, build_plan, checkpoint_layout)


def _builtin() -> None:
    """Registers the package's own architectures on first use."""
    from .. import models  # noqa: F401


def known_architectures() -> list:
    _builtin()
    return sorted(_ARCHITECTURES)


def architecture_name(raw: dict) -> str:
    """The name a config.json selects its model by: the first known entry of ``architectures``,
    else ``model_type`` at the root or under ``text_config`` (src/config.rs:350-365)."""
    _builtin()
    archs = raw.get("architectures")
    if isinstance(archs, list):
        for a in archs:
            if a in _ARCHITECTURES:
                return a
    mt = raw.get("model_type")
    if not isinstance(mt, str) and isinstance(raw.get("text_config"), dict):
        mt = raw["text_config"].get("model_type")
    if isinstance(mt, str):
        return mt
    if isinstance(archs, list) and archs:
        return str(archs[0])
    raise ConfigError("config.json has neither architectures nor model_type")


def resolve_architecture(raw: dict) -> Architecture:
    name = architecture_name(raw)
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unsupported architecture {name!r} (known: {', '.join(known_architectures())})") from None


def load_config(folder: str):
    """(architecture, typed configuration) of a model folder."""
    raw = read_config_json(folder)
    arch = resolve_architecture(raw)
    return arch, arch.config_class.from_dict(raw)
