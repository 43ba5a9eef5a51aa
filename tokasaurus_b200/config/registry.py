"""One registry from an architecture's name to its configuration class and model builder.

The reference keeps a dict from ``config.model_type`` to a model class
(tokasaurus/model/utils.py:321-327) and looks it up in ``make_model``
(tokasaurus/model/utils.py:338-340).  Here the key is the first entry of config.json's
``architectures`` list (for example ``"LlamaForCausalLM"``), with ``model_type`` as a
second way in.  An entry gives two callables: one that turns the config.json dictionary
into a typed configuration, and one that turns that configuration into a model
description made of parts (see ``tokasaurus_b200.parts.model.DecoderModel``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable


class UnknownArchitectureError(KeyError):
    pass


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[dict[str, Any]], Any]
    build_model: Callable[[Any], Any]
    model_types: tuple[str, ...] = ()


_BY_NAME: dict[str, Architecture] = {}
_BY_MODEL_TYPE: dict[str, Architecture] = {}


def register_architecture(
    name: str,
    parse_config: Callable[[dict[str, Any]], Any],
    build_model: Callable[[Any], Any],
    model_types: tuple[str, ...] = (),
    replace: bool = False,
) -> Architecture:
    """Add an architecture.  ``name`` is what config.json lists under ``architectures``."""
    if name in _BY_NAME and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    arch = Architecture(name, parse_config, build_model, tuple(model_types))
    _BY_NAME[name] = arch
    for mt in model_types:
        _BY_MODEL_TYPE[mt] = arch
    return arch


def unregister_architecture(name: str) -> None:
    arch = _BY_NAME.pop(name, None)
    if arch is not None:
        for mt in arch.model_types:
            if _BY_MODEL_TYPE.get(mt) is arch:
                del _BY_MODEL_TYPE[mt]


def known_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_BY_NAME)


def lookup_architecture(config_dict: dict[str, Any]) -> Architecture:
    """Find the architecture that a config.json dictionary names."""
    _ensure_builtin()
    for name in config_dict.get("architectures") or ():
        if name in _BY_NAME:
            return _BY_NAME[name]
    mt = config_dict.get("model_type")
    if mt in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[mt]
    raise UnknownArchitectureError(
        f"config.json names architectures={config_dict.get('architectures')!r}, "
        f"model_type={mt!r}; known architectures: {sorted(_BY_NAME)}"
    )


_builtin_loaded = False


def _ensure_builtin() -> None:
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        from tokasaurus_b200.models import llama  # noqa: F401  (registers itself)
