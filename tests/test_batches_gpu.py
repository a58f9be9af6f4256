"""Decode steps of more than eight requests, through the captured graphs, against the plain implementation.

A step's kernels change with its number of rows: up to 8 rows the weight-streaming product with one token tile, 9 to 16
with two, 17 to 127 the library's product with norm, rotary encoding and activation as kernels of their own, and the
split-key attention changes shape once (request, key/value head) pairs outnumber the SMs.  Every one of these runs here
as a replayed CUDA graph for 24 steps; the tokens are given, so every step's logits have a reference, in 32-bit and
in bfloat16.
"""

from __future__ import annotations

import pytest
import torch

import plain_llama
import tiny_configs

pytestmark = pytest.mark.gpu

# four key/value heads of 64: 40 requests make 160 (request, head) pairs, more than the SMs of the GPU
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 300, "hidden_size": 512, "intermediate_size": 328,
    "num_hidden_layers": 2, "num_attention_heads": 8, "num_key_value_heads": 4, "max_position_embeddings": 160,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "hidden_act": "silu",
}
CONFIGS = {"b": (tiny_configs.TINY_B, 2), "c": (tiny_configs.TINY_C, 4), "e": (TINY_E, 8)}
NEW = 24


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,requests", [("c", 12), ("c", 24), ("c", 64), ("b", 12), ("b", 24), ("b", 64), ("e", 40), ("e", 16)])
def test_decode_steps_of_many_requests_through_graphs(name, requests, dtype, model_folder):
    from llmserve_triton_kernels_b200 import LLM, ops
    from llmserve_triton_kernels_b200.engine.batch import StepEntry

    cfg, seed = CONFIGS[name]
    storage = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = model_folder(cfg, seed, storage)
    plain_cfg, w = plain_llama.read_model(folder)
    limit = cfg["max_position_embeddings"]
    g = torch.Generator().manual_seed(1000 + requests)
    prompt_lens = torch.randint(1, limit - NEW - 40, (requests,), generator=g).tolist()
    prompt_lens[:4] = [1, 2, 16, 17]  # the shortest contexts and a page's edge are always there
    seqs = tiny_configs.seeded_tokens(cfg["vocab_size"], [n + NEW for n in prompt_lens], 2000 + requests)
    page = 8 if name == "b" else 16
    pages = sum(-(-len(s) // page) for s in seqs) + 4
    llm = LLM(folder, dtype=dtype, device="cuda:0", block_size=page, num_blocks=pages, max_batch_size=requests,
              max_num_batched_tokens=8192)
    step = llm.step_function
    assert step.use_graphs
    names = [f"r{i}" for i in range(requests)]
    for i in range(0, requests, 16):  # prompts, all but their last token (which the first decode step brings)
        entries = [StepEntry(n, s[: p - 1], []) for n, s, p in zip(names[i : i + 16], seqs[i : i + 16], prompt_lens[i : i + 16]) if p > 1]
        if entries:
            step(entries)
    refs = [plain_llama.forward(plain_cfg, w, s) for s in seqs]
    rtol = 2e-5 if dtype == "float32" else 2e-2
    worst = 0.0
    for k in range(NEW + 1):
        entries = [StepEntry(n, [s[p - 1 + k]], [0]) for n, s, p in zip(names, seqs, prompt_lens)]
        logits = step(entries).float().cpu()
        assert step.last_was_graph, "the decode step did not replay a graph"
        for r in range(requests):
            ref = refs[r][prompt_lens[r] - 1 + k]
            diff = float((logits[r] - ref).abs().max())
            tol = rtol * float(ref.abs().max())
            assert diff <= tol, f"decode step {k}, request {r} (context {prompt_lens[r] + k}): max |diff| {diff:.3e} > {tol:.3e}"
            worst = max(worst, diff / tol)
    assert requests in step.graphs
    ops.check_device_errors()
    print(f"worst row at {worst:.2f} of the tolerance")
