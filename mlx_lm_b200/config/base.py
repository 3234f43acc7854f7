"""Typed model configurations read from ``config.json``.

A configuration class is a dataclass whose fields are the architecture's own
``config.json`` keys.  ``from_dict`` keeps the keys that are fields and drops
the rest, as ``BaseModelArgs.from_dict`` of mlx-lm does
(mlx_lm/models/base.py:11-21), but names every missing required key in one
``ValueError`` instead of failing inside the dataclass constructor.
"""

from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Dict


class ConfigError(ValueError):
    pass


@dataclasses.dataclass
class BaseModelArgs:
    @classmethod
    def from_dict(cls, params: Dict[str, Any]):
        fields = {f.name: f for f in dataclasses.fields(cls)}
        missing = [n for n, f in fields.items()
                   if n not in params and f.default is dataclasses.MISSING
                   and f.default_factory is dataclasses.MISSING]
        if missing:
            raise ConfigError(f"{cls.__module__}.{cls.__name__}: config.json lacks required key(s): "
                              + ", ".join(missing))
        args = cls(**{k: v for k, v in params.items() if k in fields})
        args.validate()
        return args

    def validate(self) -> None:  # overridden per architecture
        pass

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


def _positive_int(name: str, v) -> None:
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config key {name!r} must be a positive integer, got {v!r}")


def load_config(model_path: str) -> Dict[str, Any]:
    """``config.json`` of a model folder; end-of-sequence ids of a
    ``generation_config.json`` beside it take precedence
    (mlx_lm/utils.py:277-293)."""
    path = os.path.join(model_path, "config.json")
    if not os.path.exists(path):
        raise FileNotFoundError(f"config.json not found in {model_path}")
    with open(path) as f:
        config = json.load(f)
    gen = os.path.join(model_path, "generation_config.json")
    if os.path.exists(gen):
        try:
            with open(gen) as f:
                g = json.load(f)
        except json.JSONDecodeError:
            g = {}
        if "eos_token_id" in g:
            config["eos_token_id"] = g["eos_token_id"]
    return config
