"""Makes ``tests/golden/tiny_{a,b}.npz``: outputs of the reference's own model code on the CPU.

Run once, where the reference's sources are at hand:

    LLMSERVE_REFERENCE_SRC=<reference>/src python tests/golden/make_golden.py

For each tiny configuration it writes a model folder with this repository's random-weights
mode (32-bit storage), loads that folder with the reference's own loader
(``llmserve.weights.load_model``, float32, CPU), and stores for every prompt the reference's
full-forward logits, its greedy continuation through ``llmserve.engine.generate.generate`` and
through ``ContinuousBatchingEngine`` over a pool so small that it preempts.  A checksum of the
weights is stored too, so a later run can tell "the weights changed" from "the arithmetic
changed".  ``tests/test_plain.py`` compares the plain implementation with these files.
"""

from __future__ import annotations

import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, os.environ["LLMSERVE_REFERENCE_SRC"])

from llmserve.datatypes import SamplingParams  # noqa: E402  (the reference)
from llmserve.engine.generate import generate  # noqa: E402
from llmserve.kvcache.paged import PagedKVCache  # noqa: E402
from llmserve.scheduler.engine import ContinuousBatchingEngine  # noqa: E402
from llmserve.weights import load_model  # noqa: E402

import tiny_configs  # noqa: E402
from llmserve_triton_kernels_b200.config import LlamaConfig  # noqa: E402
from llmserve_triton_kernels_b200.weights import write_random_model  # noqa: E402

NEW_TOKENS = 16


def weights_checksum(folder) -> float:
    """Sum of |w| over the tensors of the written file (what ``tests/test_plain.py`` recomputes)."""
    from safetensors.torch import load_file

    return float(sum(t.double().abs().sum() for t in load_file(str(Path(folder) / "model.safetensors")).values()))


def main() -> None:
    for name, (cfg, seed, _, _) in tiny_configs.TINY.items():
        with tempfile.TemporaryDirectory() as tmp:
            write_random_model(tmp, LlamaConfig.from_dict(cfg), seed=seed, std=0.02, dtype=torch.float32)
            model = load_model(tmp, device="cpu", dtype=torch.float32)
            out = {"checksum": np.float64(weights_checksum(tmp))}
        prompts = tiny_configs.prompts(name)
        params = SamplingParams(temperature=0.0, max_new_tokens=NEW_TOKENS)
        with torch.inference_mode():
            for i, p in enumerate(prompts):
                out[f"prompt_{i}"] = np.asarray(p, dtype=np.int64)
                out[f"logits_{i}"] = model(torch.tensor([p]))[0].numpy()
                out[f"greedy_{i}"] = np.asarray(generate(model, p, params, device="cpu").tokens, dtype=np.int64)
        # continuous batching over a pool that forces preemption; greedy tokens must not change
        cache = PagedKVCache(model.config, num_blocks=18, block_size=4, device="cpu", dtype=torch.float32)
        engine = ContinuousBatchingEngine(model, cache, max_batch_size=3)
        ids = [engine.add_request(p, params) for p in prompts]
        done = engine.run_until_complete()
        for i, rid in enumerate(ids):
            out[f"batched_{i}"] = np.asarray(done[rid].generated, dtype=np.int64)
        out["preemptions"] = np.int64(engine.stats.preemptions)
        np.savez_compressed(HERE / f"tiny_{name}.npz", **out)
        print(name, "preemptions", engine.stats.preemptions, "checksum", out["checksum"])


if __name__ == "__main__":
    main()
