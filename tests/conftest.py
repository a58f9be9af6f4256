"""Test configuration: the ``gpu`` marker, import paths, and model folders made on the fly."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_folder(tmp_path_factory):
    """``model_folder(config_dict, seed, storage_dtype) -> Path`` of a random model, cached per session."""
    import llmserve_triton_kernels_b200.models  # noqa: F401  registers the architecture
    from llmserve_triton_kernels_b200.config import architecture_of
    from llmserve_triton_kernels_b200.weights import write_random_model

    made = {}

    def make(cfg: dict, seed: int, dtype=torch.float32, std: float = 0.02):
        key = (repr(sorted(cfg.items(), key=str)), seed, dtype, std)
        if key not in made:
            path = tmp_path_factory.mktemp("model")
            config = architecture_of(cfg).config_class.from_dict(cfg)
            made[key] = write_random_model(path, config, seed=seed, std=std, dtype=dtype)
        return made[key]

    return make


@pytest.fixture
def plain_ops_engine(monkeypatch):
    """Replaces every device operation by its plain torch statement, so that the engine's host
    logic runs on the CPU.  The engine itself has no CPU path; this is a test device only."""
    import plain_ops
    from llmserve_triton_kernels_b200 import ops

    for name in plain_ops.ALL:
        monkeypatch.setattr(ops, name, getattr(plain_ops, name))
    return ops
