"""One registry: architecture name (``model_type`` of config.json) -> how to
configure and build it.

mlx-lm resolves ``model_type`` to a module ``mlx_lm.models.<model_type>`` that
exports ``Model`` and ``ModelArgs`` (mlx_lm/utils.py:177-195).  Here an
architecture is a pair ``(args class, builder)``; the builder turns a typed
configuration into a ``ModelDescription`` (parts per layer and the order in
which layers run, see ``mlx_lm_b200.parts.model``).  Architectures that ship
with the package live in ``mlx_lm_b200.models`` and register themselves when
that package is imported; anyone else may call ``register_architecture``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Tuple, Type

from .base import BaseModelArgs, ConfigError

# aliases, as MODEL_REMAPPING in mlx_lm/utils.py:46-57 (none needed so far)
MODEL_REMAPPING: Dict[str, str] = {}


@dataclass(frozen=True)
class Architecture:
    model_type: str
    args_class: Type[BaseModelArgs]
    build: Callable  # (args) -> parts.model.ModelDescription


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(model_type: str, args_class: Type[BaseModelArgs], build: Callable,
                          replace: bool = False) -> None:
    if model_type in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {model_type!r} is already registered")
    _ARCHITECTURES[model_type] = Architecture(model_type, args_class, build)


def get_architecture(config: dict) -> Architecture:
    """The architecture a config.json names; ``ValueError`` for an unknown
    one, worded as mlx-lm words it (mlx_lm/utils.py:189-193)."""
    import mlx_lm_b200.models  # noqa: F401  (registers the built-in architectures)

    if "model_type" not in config:
        raise ConfigError("config.json lacks required key(s): model_type")
    model_type = MODEL_REMAPPING.get(config["model_type"], config["model_type"])
    arch = _ARCHITECTURES.get(model_type)
    if arch is None:
        raise ConfigError(f"Model type {model_type} not supported. Known: {sorted(_ARCHITECTURES)}")
    return arch


def get_model_classes(config: dict) -> Tuple[Callable, Type[BaseModelArgs]]:
    """``(builder, args class)`` — the shape of mlx-lm's ``_get_classes``."""
    arch = get_architecture(config)
    return arch.build, arch.args_class


def registered_architectures():
    import mlx_lm_b200.models  # noqa: F401

    return sorted(_ARCHITECTURES)
