"""Generation through the Python entry point and the command line on the GPU, against the plain
implementation: greedy tokens in 32-bit (exact) and bfloat16 (first tokens, then closeness of
logits), long decoding up to the model's last position, the first tokens of a sequence,
temperature sampling, and a model of TinyLlama's layer sizes in true 32-bit."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_llama
import tiny_configs

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def engine(folder, dtype, **opts):
    from llmserve_triton_kernels_b200 import LLM

    kw = dict(dtype=dtype, device="cuda:0", block_size=8, num_blocks=64, max_batch_size=4, max_num_batched_tokens=48, chunk_size=16)
    kw.update(opts)
    return LLM(folder, **kw)


@pytest.mark.parametrize("name", ["a", "b"])
def test_greedy_generation_float32_is_token_exact(name, model_folder):
    from llmserve_triton_kernels_b200 import SamplingParams

    cfg, seed, _, _ = tiny_configs.TINY[name]
    folder = model_folder(cfg, seed, torch.float32)
    plain_cfg, w = plain_llama.read_model(folder)
    prompts = tiny_configs.prompts(name)
    llm = engine(folder, "float32")
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=16))
    for out, prompt in zip(outs, prompts):
        assert out.token_ids == plain_llama.generate(plain_cfg, w, prompt, 16)
    # and again under pressure: so few pages that requests are preempted and recomputed
    tight = engine(folder, "float32", block_size=4, num_blocks=max(16, (max(map(len, prompts)) + 16) // 4 + 3))
    outs = tight.generate(prompts, SamplingParams(max_new_tokens=16))
    assert tight.scheduler.stats.preemptions > 0
    for out, prompt in zip(outs, prompts):
        assert out.token_ids == plain_llama.generate(plain_cfg, w, prompt, 16)
    assert tight.cache.num_free_pages == tight.cache.num_pages


@pytest.mark.parametrize("name", ["a", "b"])
def test_temperature_sampling_matches_the_plain_sampler(name, model_folder):
    from llmserve_triton_kernels_b200 import SamplingParams

    cfg, seed, _, _ = tiny_configs.TINY[name]
    folder = model_folder(cfg, seed, torch.float32)
    plain_cfg, w = plain_llama.read_model(folder)
    prompts = tiny_configs.prompts(name)
    llm = engine(folder, "float32")
    for temperature, top_k, top_p in ((0.8, 0, 1.0), (1.3, 7, 0.85)):
        outs = llm.generate(prompts, SamplingParams(max_new_tokens=16, temperature=temperature, top_k=top_k, top_p=top_p, seed=31))
        for out, prompt in zip(outs, prompts):
            assert out.token_ids == plain_llama.generate(plain_cfg, w, prompt, 16, temperature=temperature, top_k=top_k, top_p=top_p, seed=31)


@pytest.mark.parametrize("name", ["a", "b"])
def test_bfloat16_generation_follows_the_plain_one(name, model_folder):
    """bfloat16 may flip a near-tie, after which the continuations differ; so the engine's own
    tokens are fed to the plain implementation and the logits compared along them."""
    from llmserve_triton_kernels_b200 import SamplingParams
    from llmserve_triton_kernels_b200.engine.batch import StepEntry

    cfg, seed, _, _ = tiny_configs.TINY[name]
    folder = model_folder(cfg, seed, torch.bfloat16)
    plain_cfg, w = plain_llama.read_model(folder)
    prompts = tiny_configs.prompts(name)
    llm = engine(folder, "bfloat16")
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=16))
    for out, prompt in zip(outs, prompts):
        ref = plain_llama.forward(plain_cfg, w, prompt + out.token_ids)
        for i, tok in enumerate(out.token_ids):
            row = ref[len(prompt) - 1 + i]
            # the chosen token's logit is within bfloat16 error of the plain maximum
            assert float(row.max() - row[tok]) <= 2e-2 * float(row.abs().max())
    # decode-only steps ran as CUDA graphs
    assert llm.step_function.graphs, "no decode step was captured"


@pytest.mark.parametrize("name", ["a", "b"])
def test_requests_that_end_while_the_engine_runs_ahead_of_the_host(name, model_folder):
    """Decode steps are launched one step before the host reads the tokens of the step before.  Requests that end
    at different steps — by an end-of-sequence token, which the host learns a step late (the request has done a
    step too many by then, whose token must be dropped), and by different lengths — must give what the plain
    implementation gives, and every page must come back."""
    from llmserve_triton_kernels_b200 import SamplingParams

    cfg, seed, _, _ = tiny_configs.TINY[name]
    folder = model_folder(cfg, seed, torch.float32)
    plain_cfg, w = plain_llama.read_model(folder)
    prompts = tiny_configs.prompts(name)
    llm = engine(folder, "float32")
    assert llm.scheduler.run_ahead
    free = plain_llama.generate(plain_cfg, w, prompts[0], 12)
    params, want = [], []
    for i, prompt in enumerate(prompts):
        if i == 0:  # ends by the token it would choose sixth
            eos = free[5]
            params.append(SamplingParams(max_new_tokens=12, eos_token_id=eos))
            want.append(plain_llama.generate(plain_cfg, w, prompt, 12, eos=eos))
            assert want[-1][-1] == eos and len(want[-1]) <= 6
        else:  # end by lengths of their own
            params.append(SamplingParams(max_new_tokens=3 + 4 * i))
            want.append(plain_llama.generate(plain_cfg, w, prompt, 3 + 4 * i))
    outs = llm.generate(prompts, params)
    assert [o.token_ids for o in outs] == want
    assert outs[0].finish_reason == "stop" and all(o.finish_reason == "length" for o in outs[1:])
    assert llm.cache.num_free_pages == llm.cache.num_pages
    # and once more on the same engine: nothing of the last run's step too many is left over
    outs = llm.generate(prompts, params)
    assert [o.token_ids for o in outs] == want
    assert llm.cache.num_free_pages == llm.cache.num_pages


@pytest.mark.parametrize("name,stream_seed", [("a", 0), ("b", 1), ("a", 2)])
def test_requests_that_come_go_and_are_put_back_at_random(name, stream_seed, model_folder):
    """A stream of requests driven step by step: they arrive while others decode (so graph steps that run ahead of the
    host alternate with mixed steps), some are aborted, pages are so few that the newest request is put back and
    computed again, half of them sample.  What every request that is not aborted generates is what the plain
    implementation generates for it alone, and in the end every page is free."""
    import random

    from llmserve_triton_kernels_b200 import SamplingParams

    cfg, seed, _, _ = tiny_configs.TINY[name]
    folder = model_folder(cfg, seed, torch.float32)
    plain_cfg, w = plain_llama.read_model(folder)
    rng = random.Random(stream_seed)
    llm = engine(folder, "float32", num_blocks=9, max_batch_size=3, max_num_batched_tokens=24, chunk_size=8)
    sched = llm.scheduler
    assert sched.run_ahead
    arrivals = []  # (step at which it arrives, prompt, params)
    for i in range(10):
        prompt = [rng.randrange(cfg["vocab_size"]) for _ in range(rng.randint(2, 24))]
        new = rng.randint(4, 24)
        sampled = i % 2 == 1
        params = SamplingParams(max_new_tokens=new, temperature=0.9 if sampled else 0.0, top_k=rng.choice([0, 6]) if sampled else 0,
                                top_p=rng.choice([1.0, 0.9]) if sampled else 1.0, seed=100 + i)
        arrivals.append((rng.randint(0, 14), prompt, params))
    arrivals.sort(key=lambda a: a[0])
    abort_at = {arrivals[3][0] + 2: 3, arrivals[7][0] + 1: 7}  # step -> which arrival is aborted then
    ids, preempted_before, step_no = {}, sched.stats.preemptions, 0
    while step_no < 400 and (len(ids) < len(arrivals) or sched.has_unfinished()):
        for i, (at, prompt, params) in enumerate(arrivals):
            if at == step_no:
                ids[i] = sched.add_request(prompt, params)
        if step_no in abort_at and abort_at[step_no] in ids:
            sched.abort(ids[abort_at[step_no]])
        sched.step()
        step_no += 1
    assert not sched.has_unfinished()
    aborted = 0
    for i, (at, prompt, params) in enumerate(arrivals):
        r = sched.finished[ids[i]]
        if r.finish_reason == "abort":
            aborted += 1
            continue
        want = plain_llama.generate(plain_cfg, w, prompt, params.max_new_tokens, temperature=params.temperature, top_k=params.top_k,
                                    top_p=params.top_p, seed=params.seed)
        assert r.generated == want, f"request {i}"
    assert aborted <= 2
    assert sched.stats.preemptions > preempted_before  # the pages were few enough
    assert llm.cache.num_free_pages == llm.cache.num_pages
    llm.cache.check()


def test_long_decoding_to_the_last_position(model_folder):
    """One token at a time from position 1 to the model's limit, in both dtypes."""
    from llmserve_triton_kernels_b200.engine.batch import StepEntry

    cfg, seed, _, _ = tiny_configs.TINY["a"]
    limit = cfg["max_position_embeddings"]
    tokens = tiny_configs.seeded_tokens(cfg["vocab_size"], [limit], 41)[0]
    for dtype, storage, rtol in (("float32", torch.float32, 2e-5), ("bfloat16", torch.bfloat16, 2e-2)):
        folder = model_folder(cfg, seed, storage)
        plain_cfg, w = plain_llama.read_model(folder)
        ref = plain_llama.forward(plain_cfg, w, tokens)
        llm = engine(folder, dtype, block_size=16, num_blocks=limit // 16 + 1)
        for i, tok in enumerate(tokens):
            logits = llm.step_function([StepEntry("long", [tok], [0])]).float().cpu()[0]
            tol = rtol * float(ref[i].abs().max())
            assert float((logits - ref[i]).abs().max()) <= tol, f"{dtype}: position {i}"
        with pytest.raises(ValueError, match="positions"):
            llm.step_function([StepEntry("long", [1], [0])])


def test_first_tokens_of_a_sequence(model_folder):
    """Positions 0, 1, 2 alone and together: the smallest contexts a kernel sees."""
    from llmserve_triton_kernels_b200.engine.batch import StepEntry

    cfg, seed, _, _ = tiny_configs.TINY["b"]
    tokens = tiny_configs.seeded_tokens(cfg["vocab_size"], [3], 42)[0]
    for dtype, storage, rtol in (("float32", torch.float32, 2e-5), ("bfloat16", torch.bfloat16, 2e-2)):
        folder = model_folder(cfg, seed, storage)
        plain_cfg, w = plain_llama.read_model(folder)
        ref = plain_llama.forward(plain_cfg, w, tokens)
        llm = engine(folder, dtype)
        together = llm.step_function([StepEntry("t", tokens, [0, 1, 2])]).float().cpu()
        singly = torch.cat([llm.step_function([StepEntry("s", [t], [0])]).float().cpu() for t in tokens])
        for got in (together, singly):
            assert float((got - ref).abs().max()) <= rtol * float(ref.abs().max())


def test_model_of_tinyllama_layer_sizes_in_true_32_bit(model_folder):
    """Two layers of TinyLlama 1.1B's sizes (hidden 2048, 32 heads, 4 key/value heads, head size 64,
    feed-forward 5632, vocabulary 32000): whole, and the last tokens one by one."""
    from llmserve_triton_kernels_b200.config.presets import PRESETS
    from llmserve_triton_kernels_b200.engine.batch import StepEntry

    cfg = {**PRESETS["tinyllama-1.1b"], "num_hidden_layers": 2}
    folder = model_folder(cfg, 0, torch.bfloat16)
    plain_cfg, w = plain_llama.read_model(folder)
    tokens = tiny_configs.seeded_tokens(cfg["vocab_size"], [150], 43)[0]
    ref = plain_llama.forward(plain_cfg, w, tokens)
    llm = engine(folder, "float32", block_size=16, num_blocks=16, max_num_batched_tokens=256)
    whole = llm.step_function([StepEntry("w", tokens, list(range(150)))]).float().cpu()
    assert float((whole - ref).abs().max()) <= 2e-5 * float(ref.abs().max())
    llm.cache.free_request("w")
    head = llm.step_function([StepEntry("d", tokens[:140], [139])]).float().cpu()
    tail = [llm.step_function([StepEntry("d", [t], [0])]).float().cpu() for t in tokens[140:]]
    got = torch.cat([head] + tail)
    assert float((got - ref[139:]).abs().max()) <= 2e-5 * float(ref.abs().max())
    # the same in bfloat16, through the tensor-core kernels and the decode graphs
    llm16 = engine(folder, "bfloat16", block_size=16, num_blocks=16, max_num_batched_tokens=256)
    whole16 = llm16.step_function([StepEntry("w", tokens, list(range(150)))]).float().cpu()
    assert float((whole16 - ref).abs().max()) <= 2e-2 * float(ref.abs().max())
    llm16.cache.free_request("w")
    head16 = llm16.step_function([StepEntry("d", tokens[:140], [139])]).float().cpu()
    tail16 = [llm16.step_function([StepEntry("d", [t], [0])]).float().cpu().clone() for t in tokens[140:]]
    got16 = torch.cat([head16] + tail16)
    assert float((got16 - ref[139:]).abs().max()) <= 2e-2 * float(ref.abs().max())


def test_command_line(model_folder):
    cfg, seed, _, _ = tiny_configs.TINY["a"]
    folder = model_folder(cfg, seed, torch.float32)
    plain_cfg, w = plain_llama.read_model(folder)
    prompt = [t % cfg["vocab_size"] for t in range(10, 26)]  # what the command line feeds when there is no tokenizer
    out = subprocess.run(
        [sys.executable, "-m", "llmserve_triton_kernels_b200.cli", "--model", str(folder), "--dtype", "float32",
         "--max-new-tokens", "12", "--block-size", "8", "--num-blocks", "16"],
        cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert json.loads(lines[0]) == plain_llama.generate(plain_cfg, w, prompt, 12)
    assert lines[-1].startswith("[kv_cache] ttft=") and "tok/s" in lines[-1] and "peak mem=" in lines[-1]
