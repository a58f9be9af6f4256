"""The plain implementation against the reference's own model code (stored outputs)."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest
import torch

import plain_llama
import tiny_configs

GOLDEN = Path(__file__).resolve().parent / "golden"


def _weights_checksum(cfg, w) -> float:
    total = sum(float(t.double().abs().sum()) for t in w.values())
    return total


@pytest.mark.parametrize("name", ["a", "b"])
def test_plain_matches_reference_outputs(name, model_folder):
    cfg, seed, _, _ = tiny_configs.TINY[name]
    gold = np.load(GOLDEN / f"tiny_{name}.npz")
    cfg_read, w = plain_llama.read_model(model_folder(cfg, seed, torch.float32))
    assert abs(_weights_checksum(cfg_read, w) - float(gold["checksum"])) < 1e-6 * float(gold["checksum"]), (
        "the seeded random weights differ from the ones the stored outputs were made with"
    )
    assert int(gold["preemptions"]) > 0
    for i, prompt in enumerate(tiny_configs.prompts(name)):
        assert prompt == gold[f"prompt_{i}"].tolist()
        logits = plain_llama.forward(cfg_read, w, prompt)
        torch.testing.assert_close(logits, torch.from_numpy(gold[f"logits_{i}"]), atol=1e-5, rtol=0)
        tokens = plain_llama.generate(cfg_read, w, prompt, 16)
        assert tokens == gold[f"greedy_{i}"].tolist()
        assert tokens == gold[f"batched_{i}"].tolist()


def test_plain_window_and_schedule_are_consistent(model_folder):
    cfg, seed, _, _ = tiny_configs.TINY["a"]
    cfg_read, w = plain_llama.read_model(model_folder(cfg, seed, torch.float32))
    tokens = tiny_configs.seeded_tokens(cfg["vocab_size"], [40], 7)[0]
    full = plain_llama.forward(cfg_read, w, tokens)
    # a window as long as the sequence changes nothing; a short one changes late positions only
    same = plain_llama.forward(cfg_read, w, tokens, windows=[40, 40])
    torch.testing.assert_close(full, same, atol=1e-6, rtol=0)
    short = plain_llama.forward(cfg_read, w, tokens, windows=[8, None])
    torch.testing.assert_close(full[:8], short[:8], atol=1e-6, rtol=0)
    assert (full[8:] - short[8:]).abs().max() > 1e-4


def test_uniform_is_in_range_and_reproducible():
    us = [plain_llama.uniform_from(1234, n) for n in range(1000)]
    assert all(0.0 <= u < 1.0 for u in us)
    assert us == [plain_llama.uniform_from(1234, n) for n in range(1000)]
    assert abs(sum(us) / len(us) - 0.5) < 0.05
    assert len(set(us)) > 990
