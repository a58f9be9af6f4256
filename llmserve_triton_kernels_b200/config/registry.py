"""One registry from an architecture's name (config.json ``architectures[0]``) to its model.

An architecture is a configuration class that reads its own config.json keys and a function
that turns such a configuration into a :class:`ModelPlan` (layers from parts, and the order in
which they run).  The reference has no registry: its loader hard-codes one class
(src/llmserve/weights.py:46) and never reads ``architectures``.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any  # has from_dict(dict) and to_dict()
    plan: Callable[[Any], Any]  # config -> ModelPlan
    model_class: Any = None  # a subclass of models.model.Model (None: Model itself)


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class, plan, model_class=None) -> Architecture:
    """``model_class``: a subclass of ``Model`` for an architecture that prepares its embeddings or treats its
    logits in a way of its own (``Model.embed_tokens``, ``Model.project_logits``); most need none."""
    arch = Architecture(name, config_class, plan, model_class)
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise KeyError(
            f"architecture {name!r} is not registered; known architectures: {known_architectures()}"
        )
    return _ARCHITECTURES[name]


def architecture_of(config_dict: dict) -> Architecture:
    names = config_dict.get("architectures")
    if not names or not isinstance(names, (list, tuple)):
        raise KeyError(
            "config.json has no 'architectures' list, so the model class cannot be chosen; "
            f"known architectures: {known_architectures()}"
        )
    return get_architecture(names[0])


def read_config(model_dir: str | Path):
    """``(architecture, typed configuration)`` of the model folder."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path} does not exist: a model folder holds config.json and *.safetensors")
    d = json.loads(path.read_text())
    arch = architecture_of(d)
    return arch, arch.config_class.from_dict(d)
