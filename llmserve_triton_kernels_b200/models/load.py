"""From a model folder, or from a configuration and a seed, to a bound :class:`Model`."""

from __future__ import annotations

from pathlib import Path

import torch

from ..config.registry import get_architecture, read_config
from ..weights.loader import check_tensors, read_safetensors
from ..weights.random_init import random_tensors
from .model import Model

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in DTYPES.values():
            raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {dtype}")
        return dtype
    if dtype not in DTYPES:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {dtype!r}")
    return DTYPES[dtype]


def load_model(model_dir: str | Path, dtype="bfloat16", device="cuda:0"):
    """``(model, configuration)`` of the folder; the model class follows config.json's ``architectures``."""
    arch, config = read_config(model_dir)
    model = (arch.model_class or Model)(arch.plan(config), resolve_dtype(dtype), device)
    tensors = read_safetensors(model_dir)
    check_tensors(tensors, model.tensor_specs(), model.ignored_tensor_names(), where=str(model_dir))
    model.bind(tensors)
    return model, config


def random_model(config, seed: int, dtype="bfloat16", device="cuda:0", std: float = 0.02, storage=torch.bfloat16):
    """The model that :func:`write_random_model` would write and :func:`load_model` read back, without the disk."""
    arch = get_architecture(config.architecture)
    model = (arch.model_class or Model)(arch.plan(config), resolve_dtype(dtype), device)
    model.bind(random_tensors(model.tensor_specs(), seed, std, storage))
    return model
