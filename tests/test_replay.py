"""Trace replay in every way of cutting the work, against the plain implementation.

The same requests are replayed whole, with the last 32 tokens decoded one by one, in portions
of changing size, and mixed with other requests over a pool so small that pages are used
again.  On the GPU ``bin/trace_run`` runs as a user would start it, in 32-bit and in bfloat16;
without a GPU the same traces go through the replay program in-process with the plain
operations patched in, which checks the host side (cache, batches, step function).
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_llama
import tiny_configs
import trace_tools

F32_RTOL = 2e-5  # of the largest |logit| of the row's reference; the arithmetic is all 32-bit
BF16_RTOL = 2e-2  # bfloat16 keeps 8 bits: ~20 roundings of ~2^-9 between the tokens and the logits


def tolerance(dtype: str):
    r = F32_RTOL if dtype == "float32" else BF16_RTOL
    return lambda ref: r * max(float(np.abs(ref).max()), 1e-3)


def requests_for(name: str) -> dict[str, list[int]]:
    """The configuration's prompts, each followed by 34 given tokens, and one long request."""
    cfg, _, prompt_seed, lens = tiny_configs.TINY[name]
    vocab, limit = cfg["vocab_size"], cfg["max_position_embeddings"]
    seqs = tiny_configs.seeded_tokens(vocab, [n + 34 for n in lens] + [limit - 3], prompt_seed + 100)
    return {f"r{i}": s for i, s in enumerate(seqs)}


def all_modes(name: str) -> tuple[trace_tools.Trace, dict[str, list[int]]]:
    """One trace holding the four ways, request names tagged by way."""
    reqs = requests_for(name)
    trace = trace_tools.Trace()
    flat: dict[str, list[int]] = {}
    for req, tokens in reqs.items():
        for tag, make in (("w", trace_tools.whole), ("d", trace_tools.decode_tail), ("p", trace_tools.portions)):
            trace.extend(make(f"{tag}.{req}", tokens))
            flat[f"{tag}.{req}"] = tokens
    short = {f"m.{r}": t for r, t in list(reqs.items())[:-1]}
    # twice through, so that the second round runs on pages that the first one gave back
    both = {**short, **{k + "'": v for k, v in short.items()}}
    prefill = {k: len(v) - 34 for k, v in both.items()}
    trace.extend(trace_tools.mixed(both, prefill, chunk=16, live=4))
    flat.update(both)
    return trace, flat


def expected_logits(model_dir, flat):
    cfg, w = plain_llama.read_model(model_dir)
    cache: dict[tuple, torch.Tensor] = {}
    out = {}
    for req, tokens in flat.items():
        key = tuple(tokens)
        if key not in cache:
            cache[key] = plain_llama.forward(cfg, w, tokens)
        out[req] = cache[key]
    return out


@pytest.mark.parametrize("name", ["a", "b"])
def test_replay_host_logic_with_plain_operations(name, model_folder, tmp_path, plain_ops_engine):
    cfg, seed, _, _ = tiny_configs.TINY[name]
    folder = model_folder(cfg, seed, torch.float32)
    trace, flat = all_modes(name)
    got = trace_tools.run_trace_inprocess(folder, "float32", trace, tmp_path, page_size=8 if name == "b" else 16)
    assert len(got) == sum(len(v) for v in trace.rows.values())
    trace_tools.compare(got, expected_logits(folder, flat), tolerance("float32"))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_replay_on_gpu(name, dtype, model_folder, tmp_path):
    cfg, seed, _, _ = tiny_configs.TINY[name]
    storage = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = model_folder(cfg, seed, storage)
    trace, flat = all_modes(name)
    got = trace_tools.run_trace(folder, dtype, trace, tmp_path, page_size=8 if name == "b" else None)
    assert len(got) == sum(len(v) for v in trace.rows.values())
    worst = trace_tools.compare(got, expected_logits(folder, flat), tolerance(dtype))
    print(f"worst row (fraction of tolerance, (request, position, diff)): {worst}")


def _edges(pos: int) -> bool:
    """Every fifth position, and the edges of pages, key tiles and query tiles."""
    return pos % 5 == 0 or pos % 16 in (0, 15) or pos % 64 in (0, 1, 63)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("preset", ["tinyllama-1.1b", "llama2-7b", "llama3-8b"])
def test_replay_at_real_layer_sizes(preset, dtype, model_folder, tmp_path):
    """Two layers of the sizes of TinyLlama 1.1B, Llama-2 7B (32 key/value heads of 128, feed-forward 11008) and
    Llama-3 8B (8 key/value heads, feed-forward 14336, vocabulary 128256) in the four ways of cutting: a request of 300
    tokens whole (on the tensor-core prefill kernels in bfloat16), with its last 32 tokens one by one, and in portions
    of 2 to 16 tokens; and shorter requests mixed, portions of some beside decoded tokens of others, over a pool in
    which pages are used again.  Rows are compared at every fifth position and at the edges of pages and tiles."""
    from llmserve_triton_kernels_b200.config.presets import PRESETS

    cfg = {**PRESETS[preset], "num_hidden_layers": 2, "max_position_embeddings": 512}
    folder = model_folder(cfg, 0, torch.bfloat16)
    long, short_a, short_b = tiny_configs.seeded_tokens(cfg["vocab_size"], [300, 97, 70], 77)
    late = lambda n: (lambda pos: _edges(pos) or pos >= n - 34)  # noqa: E731
    trace = trace_tools.Trace()
    flat = {}
    for tag, make in (("w", trace_tools.whole), ("d", trace_tools.decode_tail), ("p", trace_tools.portions)):
        trace.extend(make(f"{tag}.long", long, keep=late(len(long))))
        flat[f"{tag}.long"] = long
    trace.extend(trace_tools.whole("w.a", short_a, keep=late(len(short_a))))
    flat["w.a"] = short_a
    both = {"m.a": short_a, "m.b": short_b, "m.a'": short_a, "m.b'": short_b, "m.a''": short_a}
    trace.extend(trace_tools.mixed(both, {k: len(v) - 34 for k, v in both.items()}, chunk=16, live=4, keep=_edges))
    flat.update(both)
    # the smallest of the three keeps every product of 128 rows and more on the own tcgen05 kernel; the others take the
    # faster of that and the library's, as serving does
    env = {"LLMSERVE_B200_GEMM": "own"} if preset == "tinyllama-1.1b" else None
    got = trace_tools.run_trace(folder, dtype, trace, tmp_path, env=env)
    assert len(got) == sum(len(v) for v in trace.rows.values())
    worst = trace_tools.compare(got, expected_logits(folder, flat), tolerance(dtype))
    print(f"worst row (fraction of tolerance, (request, position, diff)): {worst}")


def test_replay_program_with_random_weights_of_a_named_configuration(tmp_path, plain_ops_engine):
    """``--random PRESET --seed S`` stands in for a model folder: the same weights as ``write_random_model`` writes for
    that configuration and seed, so the logits equal those of the folder's replay."""
    import io
    import json
    import sys

    from llmserve_triton_kernels_b200 import replay
    from llmserve_triton_kernels_b200.config import LlamaConfig
    from llmserve_triton_kernels_b200.config.presets import PRESETS
    from llmserve_triton_kernels_b200.weights import write_random_model

    tokens = tiny_configs.seeded_tokens(256, [9], 5)[0]
    step = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": tokens, "want": [0, 8]}], "end": ["a"]}) + "\n"
    folder = write_random_model(tmp_path / "m", LlamaConfig.from_dict(PRESETS["tiny"]), seed=3, dtype=torch.bfloat16)
    outs = []
    for name, source in (("folder", ["--model", str(folder)]), ("random", ["--random", "tiny", "--seed", "3"])):
        stdin, stdout = sys.stdin, sys.stdout
        sys.stdin, sys.stdout = io.StringIO(step), io.StringIO()
        try:
            assert replay.main([*source, "--dtype", "float32", "--out", str(tmp_path / name), "--max-tokens", "64", "--device", "cpu"]) == 0
        finally:
            sys.stdin, sys.stdout = stdin, stdout
        outs.append(np.fromfile(tmp_path / name / "0.f32", dtype="<f4"))
    assert outs[0].shape == (2 * 256,) and np.array_equal(outs[0], outs[1])
    with pytest.raises(SystemExit):
        replay.parse_args(["--out", "x", "--max-tokens", "1"])
