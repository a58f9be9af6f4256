"""Random weights from a configuration and a seed, and a model folder written from them.

The reference's ``random_model`` (src/llmserve/weights.py:60-79) draws from one generator in
module order.  Here every tensor has a generator of its own, seeded from the seed and the
tensor's name, so the values do not depend on the order or on how a part stacks its matrices.
Matrices are N(0, std); norm weights are 1 + N(0, std), so that a norm that forgot its weight
shows in the logits.
"""

from __future__ import annotations

import json
import zlib
from pathlib import Path

import torch

from ..parts.base import TensorSpec


def _generator(seed: int, name: str) -> torch.Generator:
    return torch.Generator().manual_seed((int(seed) * 1_000_003 + zlib.crc32(name.encode())) % (2**63))


def random_tensor(name: str, spec: TensorSpec, seed: int, std: float, dtype: torch.dtype) -> torch.Tensor:
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype)
    values = torch.randn(spec.shape, generator=_generator(seed, name), dtype=torch.float32) * std
    if spec.init == "ones_plus_normal":
        values = values + 1.0
    elif spec.init != "normal":
        raise ValueError(f"tensor {name!r} has an unknown init {spec.init!r}")
    return values.to(dtype)


def random_tensors(
    specs: dict[str, TensorSpec], seed: int, std: float = 0.02, dtype: torch.dtype = torch.bfloat16
) -> dict[str, torch.Tensor]:
    return {name: random_tensor(name, spec, seed, std, dtype) for name, spec in specs.items()}


def write_random_model(
    model_dir: str | Path,
    config,
    seed: int,
    std: float = 0.02,
    dtype: torch.dtype = torch.bfloat16,
) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a registered architecture's
    configuration) with weights drawn from ``seed``.  Returns the folder."""
    from safetensors.torch import save_file

    from ..config.registry import get_architecture
    from ..models.model import Model

    arch = get_architecture(config.architecture)
    model = (arch.model_class or Model)(arch.plan(config), torch.float32, "cpu")
    tensors = random_tensors(model.tensor_specs(), seed, std, dtype)
    path = Path(model_dir)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config.to_dict(), indent=1))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(path / "model.safetensors"))
    return path
