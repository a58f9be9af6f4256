"""Weights from safetensors, by tensor name.

Parity: src/llmserve/weights.py:24-57 reads every ``*.safetensors`` file of the folder, skips the
legacy ``rotary_emb.inv_freq`` buffers, and raises on missing or unexpected names.  Here the
check is explicit and complete: one error lists every missing tensor, every unexpected one
and every wrong shape.  Stored precision is kept: bfloat16 stays bfloat16, a tensor stored in
32-bit stays 32-bit (half precision becomes bfloat16, float64 becomes float32), integer tables
become int32.  The parts cast what their kernels need when they take the tensors.
"""

from __future__ import annotations

from pathlib import Path

import torch

from ..parts.base import TensorSpec

_SKIPPED_SUFFIXES = ("rotary_emb.inv_freq",)


class WeightError(RuntimeError):
    """The checkpoint does not hold the tensors the model declares."""

    def __init__(self, missing, unexpected, wrong_shape, where: str = ""):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        lines = [f"checkpoint mismatch{' in ' + where if where else ''}:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(
                f"  wrong shape ({len(self.wrong_shape)}): "
                + ", ".join(f"{n} expected {list(e)} got {list(g)}" for n, e, g in self.wrong_shape)
            )
        super().__init__("\n".join(lines))


def _stored(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32, torch.int32):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if not t.dtype.is_floating_point:
        return t.to(torch.int32)
    return t.to(torch.float32)


def read_safetensors(model_dir: str | Path) -> dict[str, torch.Tensor]:
    """Every tensor of every ``*.safetensors`` file in the folder, on the host."""
    from safetensors import safe_open

    path = Path(model_dir)
    files = sorted(path.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files found in {path}")
    tensors: dict[str, torch.Tensor] = {}
    for f in files:
        with safe_open(str(f), framework="pt", device="cpu") as sf:
            for key in sf.keys():  # noqa: SIM118
                if key.endswith(_SKIPPED_SUFFIXES):
                    continue
                tensors[key] = _stored(sf.get_tensor(key))
    return tensors


def check_tensors(
    tensors: dict[str, torch.Tensor],
    specs: dict[str, TensorSpec],
    ignored: set[str] = frozenset(),
    where: str = "",
) -> None:
    missing = [n for n, s in specs.items() if n not in tensors and not s.optional]
    unexpected = [n for n in tensors if n not in specs and n not in ignored]
    wrong = [
        (n, tuple(s.shape), tuple(tensors[n].shape))
        for n, s in specs.items()
        if n in tensors and tuple(tensors[n].shape) != tuple(s.shape)
    ]
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, where)
