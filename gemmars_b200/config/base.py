"""Typed model configurations read from a checkpoint's ``config.json``.

A configuration class lists its fields with ``key(...)``; ``ModelConfig.from_dict`` reads each
one from the JSON object under its own config.json name, checks its type, and reports every
problem of the file in one error.  No model size lives anywhere else in the package.

Reference: the serde structs of src/config.rs:383-452 and ``QwenConfig::load``
(src/config.rs:455-486), which parse the root object or its ``text_config``.
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Optional

REQUIRED = object()
_NULLABLE = ("opt_int", "str_list", "opt_dict")


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names every offending key."""


def key(kind, default=REQUIRED, *, doc=""):
    """A dataclass field read from config.json under the field's own name.

    ``kind`` is int, float, bool, str, "int_list", "str_list", "opt_int" or "opt_dict".
    """
    md = {"kind": kind, "required": default is REQUIRED, "doc": doc}
    if default is REQUIRED:
        return dataclasses.field(metadata=md)
    if isinstance(default, (list, dict)):
        return dataclasses.field(default_factory=lambda: type(default)(default), metadata=md)
    return dataclasses.field(default=default, metadata=md)


def _coerce(name, kind, value, errors):
    def bad(expect):
        errors.append(f"{name}: expected {expect}, got {value!r}")
        return None

    if kind is bool:
        return value if isinstance(value, bool) else bad("true or false")
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            return bad("an integer")
        return value
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            return bad("a number")
        return float(value)
    if kind is str:
        return value if isinstance(value, str) else bad("a string")
    if kind == "opt_int":
        if value is None:
            return None
        if isinstance(value, bool) or not isinstance(value, int):
            return bad("an integer or null")
        return value
    if kind == "int_list":  # a number or a list of numbers (eos_token_id, src/config.rs:326-332)
        if isinstance(value, int) and not isinstance(value, bool):
            return [value]
        if isinstance(value, list) and all(isinstance(v, int) and not isinstance(v, bool) for v in value):
            return list(value)
        return bad("an integer or a list of integers")
    if kind == "str_list":
        if value is None:
            return None
        if isinstance(value, list) and all(isinstance(v, str) for v in value):
            return list(value)
        return bad("a list of strings or null")
    if kind == "opt_dict":
        if value is None or isinstance(value, dict):
            return value
        return bad("an object or null")
    raise TypeError(f"unknown key kind {kind!r}")


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration."""

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json: the top level must be an object")
        # The text model's keys may sit under "text_config" (src/config.rs:462-463).
        text = raw.get("text_config") if isinstance(raw.get("text_config"), dict) else raw
        errors, values = [], {}
        for f in dataclasses.fields(cls):
            md = f.metadata
            if "kind" not in md:
                continue
            present = f.name in text or f.name in raw
            if not present:
                if md["required"]:
                    errors.append(f"{f.name}: missing")
                continue
            value = text[f.name] if f.name in text else raw[f.name]
            if value is None and not md["required"] and md["kind"] not in _NULLABLE:
                continue  # an explicit null means "default"
            got = _coerce(f.name, md["kind"], value, errors)
            if got is not None or md["kind"] in _NULLABLE:
                values[f.name] = got
        if errors:
            raise ConfigError("config.json: " + "; ".join(errors))
        cfg = cls(**values)
        problems = cfg.validate()
        if problems:
            raise ConfigError("config.json: " + "; ".join(problems))
        return cfg

    @classmethod
    def from_folder(cls, folder: str) -> "ModelConfig":
        return cls.from_dict(read_config_json(folder))

    def validate(self) -> list:
        """Problems of the values taken together (empty when the configuration is usable)."""
        return []

    def to_dict(self) -> dict:
        """The config.json object that reads back as this configuration."""
        return {f.name: getattr(self, f.name) for f in dataclasses.fields(self) if "kind" in f.metadata}


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    try:
        with open(path) as f:
            return json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: not found") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None


def load_stop_ids(folder: str, fallback: Optional[list] = None) -> list:
    """Stop tokens of a checkpoint: ``eos_token_id`` (a number or a list) from
    generation_config.json, else from config.json or its text_config (src/config.rs:322-347).
    The reference falls back to another model family's ids; here the fallback is the caller's
    (none by default)."""
    def ids(v: Any):
        if isinstance(v, int) and not isinstance(v, bool):
            return [v]
        if isinstance(v, list):
            return [x for x in v if isinstance(x, int) and not isinstance(x, bool)]
        return None

    for name in ("generation_config.json", "config.json"):
        try:
            with open(os.path.join(folder, name)) as f:
                raw = json.load(f)
        except (OSError, json.JSONDecodeError):
            continue
        found = ids(raw.get("eos_token_id"))
        if found is None and isinstance(raw.get("text_config"), dict):
            found = ids(raw["text_config"].get("eos_token_id"))
        if found is not None:
            return found
    return list(fallback or [])
