"""The scheduler's decisions, on the CPU: the device operations are replaced by their plain torch
statements (``plain_ops_engine``), so everything above the kernels is the engine's own code.

Pattern of the reference's tests (tests/test_scheduler.py there): greedy tokens must equal
independent generation whatever the batching, the cutting into portions or the preemptions, and
no page may be left held afterwards."""

from __future__ import annotations

import pytest
import torch

import plain_llama
import tiny_configs
from llmserve_triton_kernels_b200 import LLM, SamplingParams
from llmserve_triton_kernels_b200.engine.batch import StepEntry
from llmserve_triton_kernels_b200.engine.scheduler import Status


def make(model_folder, name="a", **opts):
    cfg, seed, _, _ = tiny_configs.TINY[name]
    folder = model_folder(cfg, seed, torch.float32)
    kw = dict(dtype="float32", device="cpu", block_size=4, num_blocks=64, max_batch_size=3, max_num_batched_tokens=64)
    kw.update(opts)
    return LLM(folder, **kw), plain_llama.read_model(folder)


def plain_tokens(plain, prompt, n, **kw):
    cfg, w = plain
    return plain_llama.generate(cfg, w, prompt, n, **kw)


REQUESTS = [(5, 9), (12, 6), (8, 12), (3, 7), (10, 5), (6, 10)]  # (prompt length, new tokens)


@pytest.mark.parametrize("policy", ["continuous", "static"])
def test_tokens_equal_independent_generation(model_folder, plain_ops_engine, policy):
    llm, plain = make(model_folder, policy=policy)
    prompts = tiny_configs.seeded_tokens(256, [p for p, _ in REQUESTS], 11)
    outs = llm.generate(prompts, [SamplingParams(max_new_tokens=n) for _, n in REQUESTS])
    for out, prompt, (_, n) in zip(outs, prompts, REQUESTS):
        assert out.token_ids == plain_tokens(plain, prompt, n)
        assert out.finish_reason == "length" and len(out.step_latencies_s) == n - 1
    assert llm.cache.num_free_pages == llm.cache.num_pages  # nothing leaked
    llm.cache.check()


def test_portions_under_a_token_budget_mix_with_decodes(model_folder, plain_ops_engine):
    llm, plain = make(model_folder, "b", block_size=8, num_blocks=40, max_batch_size=4, max_num_batched_tokens=24, chunk_size=16)
    prompts = tiny_configs.prompts("b")  # lengths 1, 7, 23, 40
    sched = llm.scheduler
    ids = [sched.add_request(p, SamplingParams(max_new_tokens=16)) for p in prompts]
    mixed_steps = 0
    while sched.has_unfinished():
        sched.step()
        s = sched.stats
        assert s.last_batch_tokens <= 24
        plan_has_portion = any(len(r.all_ids) - r.num_computed > 1 for r in sched.running)
        plan_has_decode = any(len(r.all_ids) - r.num_computed == 1 and r.generated for r in sched.running)
        mixed_steps += plan_has_portion and plan_has_decode
    assert mixed_steps > 0  # portions of the long prompt ran beside decoded tokens of the short ones
    for rid, prompt in zip(ids, prompts):
        assert sched.finished[rid].generated == plain_tokens(plain, prompt, 16)
    assert sched.stats.prefill_tokens == sum(map(len, prompts)) and sched.stats.preemptions == 0
    assert llm.cache.num_free_pages == llm.cache.num_pages


def test_a_request_joins_mid_flight(model_folder, plain_ops_engine):
    llm, plain = make(model_folder)
    sched = llm.scheduler
    p1, p2 = tiny_configs.seeded_tokens(256, [9, 6], 12)
    a = sched.add_request(p1, SamplingParams(max_new_tokens=12))
    for _ in range(4):
        sched.step()
    b = sched.add_request(p2, SamplingParams(max_new_tokens=5))
    sched.step()
    assert {r.req_id for r in sched.running} == {a, b}  # joined on the very next step
    sched.run_until_complete()
    assert sched.finished[a].generated == plain_tokens(plain, p1, 12)
    assert sched.finished[b].generated == plain_tokens(plain, p2, 5)


def test_static_policy_waits_for_the_batch_to_drain(model_folder, plain_ops_engine):
    llm, _ = make(model_folder, policy="static", max_batch_size=2)
    sched = llm.scheduler
    p = tiny_configs.seeded_tokens(256, [4, 4, 4], 13)
    for x in p:
        sched.add_request(x, SamplingParams(max_new_tokens=4))
    sched.step()
    assert len(sched.running) == 2 and len(sched.waiting) == 1
    sched.step()
    assert len(sched.waiting) == 1  # the third waits until the whole batch has drained
    sched.run_until_complete()
    assert len(sched.finished) == 3


def test_pages_run_out_newest_request_is_preempted_and_recomputed(model_folder, plain_ops_engine):
    llm, plain = make(model_folder, num_blocks=14, block_size=4, max_batch_size=4)
    prompts = tiny_configs.seeded_tokens(256, [6, 6, 6, 6], 14)
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=14))  # 4 x 20 tokens = 20 pages > 14
    stats = llm.scheduler.stats
    assert stats.preemptions > 0
    assert sum(o.num_preemptions for o in outs) == stats.preemptions
    for out, prompt in zip(outs, prompts):
        assert out.token_ids == plain_tokens(plain, prompt, 14)
    assert llm.cache.num_free_pages == 14
    llm.cache.check()


def test_preempted_sampling_request_keeps_its_random_stream(model_folder, plain_ops_engine):
    llm, plain = make(model_folder, num_blocks=12, block_size=4, max_batch_size=3)
    prompts = tiny_configs.seeded_tokens(256, [7, 7, 7], 15)
    params = SamplingParams(max_new_tokens=12, temperature=0.8, top_k=40, top_p=0.95, seed=123)
    outs = llm.generate(prompts, params)
    assert llm.scheduler.stats.preemptions > 0
    for out, prompt in zip(outs, prompts):
        assert out.token_ids == plain_tokens(plain, prompt, 12, temperature=0.8, top_k=40, top_p=0.95, seed=123)


def test_eos_stops_and_frees(model_folder, plain_ops_engine):
    llm, plain = make(model_folder)
    prompt = tiny_configs.seeded_tokens(256, [8], 16)[0]
    free_run = plain_tokens(plain, prompt, 10)
    eos = free_run[3]
    out = llm.generate([prompt], SamplingParams(max_new_tokens=10, eos_token_id=eos))[0]
    cut = free_run.index(eos) + 1
    assert out.token_ids == free_run[:cut] and out.finish_reason == "stop"  # the stop token is emitted
    assert llm.cache.num_free_pages == llm.cache.num_pages


def test_abort_of_waiting_and_running_requests(model_folder, plain_ops_engine):
    llm, _ = make(model_folder, max_batch_size=1)
    sched = llm.scheduler
    p = tiny_configs.seeded_tokens(256, [5, 5], 17)
    a = sched.add_request(p[0], SamplingParams(max_new_tokens=20))
    b = sched.add_request(p[1], SamplingParams(max_new_tokens=20))
    sched.step()
    sched.abort(b)  # waiting
    sched.abort(a)  # running
    events = sched.step()
    assert {(e.req_id, e.finish_reason) for e in events if e.finished} == {(a, "abort"), (b, "abort")}
    assert not sched.has_unfinished() and llm.cache.num_free_pages == llm.cache.num_pages
    assert sched.finished[a].status is Status.FINISHED
    sched.abort(a)  # already finished: ignored
    sched.step()


def test_requests_that_can_never_run_are_refused(model_folder, plain_ops_engine):
    llm, _ = make(model_folder, num_blocks=6, block_size=4)
    sched = llm.scheduler
    with pytest.raises(ValueError, match="at least one token"):
        sched.add_request([], SamplingParams())
    with pytest.raises(ValueError, match="max_new_tokens"):
        SamplingParams(max_new_tokens=0)
    with pytest.raises(ValueError, match="exceeds model limit"):
        sched.add_request([1] * 100, SamplingParams(max_new_tokens=100))
    with pytest.raises(ValueError, match="pages"):
        sched.add_request([1] * 20, SamplingParams(max_new_tokens=10))  # 8 pages needed, 6 exist
    with pytest.raises(ValueError, match="outside"):
        llm.step_function([StepEntry("x", [999], [0])])


def test_snapshot_and_seed_reproducibility(model_folder, plain_ops_engine):
    llm, _ = make(model_folder)
    prompts = tiny_configs.seeded_tokens(256, [6, 9], 18)
    params = SamplingParams(max_new_tokens=8, temperature=1.0, seed=7)
    first = [o.token_ids for o in llm.generate(prompts, params)]
    again = [o.token_ids for o in llm.generate(prompts, params)]
    other = [o.token_ids for o in llm.generate(prompts, SamplingParams(max_new_tokens=8, temperature=1.0, seed=8))]
    assert first == again and first != other
    snap = llm.scheduler.snapshot()
    assert snap["running"] == 0 and snap["free_blocks"] == snap["total_blocks"] and snap["tokens_generated"] == 48


# ------------------------------------------------------------------ one step ahead of the host
def ahead(llm):
    """On a GPU decode steps are launched before the host has read the tokens of the step before; the same logic
    runs here on the CPU (the step function then reads the tokens from the tensor, which changes nothing)."""
    llm.scheduler.run_ahead = True
    return llm


@pytest.mark.parametrize("policy", ["continuous", "static"])
def test_running_ahead_of_the_host_changes_no_token(model_folder, plain_ops_engine, policy):
    llm, plain = make(model_folder, policy=policy)
    ahead(llm)
    prompts = tiny_configs.seeded_tokens(256, [p for p, _ in REQUESTS], 11)
    outs = llm.generate(prompts, [SamplingParams(max_new_tokens=n) for _, n in REQUESTS])
    for out, prompt, (_, n) in zip(outs, prompts, REQUESTS):
        assert out.token_ids == plain_tokens(plain, prompt, n)
        assert out.finish_reason == "length"
    assert llm.cache.num_free_pages == llm.cache.num_pages
    llm.cache.check()
    assert llm.scheduler._ahead is None


def test_running_ahead_a_stop_token_is_learnt_a_step_late(model_folder, plain_ops_engine):
    llm, plain = make(model_folder)
    ahead(llm)
    prompts = tiny_configs.seeded_tokens(256, [8, 5], 16)
    free_run = plain_tokens(plain, prompts[0], 10)
    eos = free_run[4]
    sched = llm.scheduler
    a = sched.add_request(prompts[0], SamplingParams(max_new_tokens=10, eos_token_id=eos))
    b = sched.add_request(prompts[1], SamplingParams(max_new_tokens=10))
    launched_too_many = False
    while sched.has_unfinished():
        sched.step()
        fin = sched.finished.get(a)
        if fin is not None and sched._ahead is not None and fin in sched._ahead.reqs:
            launched_too_many = True  # a's step too many is in flight; its token must never show
    assert launched_too_many
    cut = free_run.index(eos) + 1
    assert sched.finished[a].generated == free_run[:cut] and sched.finished[a].finish_reason == "stop"
    assert sched.finished[b].generated == plain_tokens(plain, prompts[1], 10)
    assert llm.cache.num_free_pages == llm.cache.num_pages
    llm.cache.check()


def test_running_ahead_with_few_pages_and_an_abort(model_folder, plain_ops_engine):
    llm, plain = make(model_folder, block_size=4, num_blocks=10, max_batch_size=3)
    ahead(llm)
    prompts = tiny_configs.seeded_tokens(256, [9, 10, 11], 12)
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=12))
    assert llm.scheduler.stats.preemptions > 0
    for out, prompt in zip(outs, prompts):
        assert out.token_ids == plain_tokens(plain, prompt, 12)
    assert llm.cache.num_free_pages == llm.cache.num_pages
    # an abort while a step is in flight ahead of the host
    sched = llm.scheduler
    a = sched.add_request(prompts[0], SamplingParams(max_new_tokens=30))
    while sched._ahead is None:
        sched.step()
    sched.abort(a)
    events = []
    while sched.has_unfinished():
        events += sched.step()
    assert [(e.req_id, e.finish_reason) for e in events if e.finished] == [(a, "abort")]
    got = sched.finished[a].generated
    assert got == plain_tokens(plain, prompts[0], 30)[: len(got)]
    assert llm.cache.num_free_pages == llm.cache.num_pages
    llm.cache.check()


def test_a_kernel_that_reports_a_failed_wait_stops_the_engine(model_folder, plain_ops_engine, monkeypatch):
    """Kernels whose bounded waits give up set a word in pinned host memory and run to their end with invalid
    results.  The scheduler reads the word wherever it has just waited for the device: the step's tokens are not
    handed out, everything in flight is dropped with its pages, and the error is raised.  The word is set from the
    host here; no kernel is made to fail."""
    from llmserve_triton_kernels_b200 import ops

    llm, plain = make(model_folder)
    sched = llm.scheduler
    prompts = tiny_configs.seeded_tokens(256, [6, 9], 19)
    ids = [sched.add_request(p, SamplingParams(max_new_tokens=8)) for p in prompts]
    sched.step()
    sched.step()
    flag = torch.zeros(1, dtype=torch.int32)
    monkeypatch.setattr(ops, "_error_flag", flag)
    flag[0] = 1
    with pytest.raises(ops.KernelError, match="wait"):
        sched.step()
    assert int(flag[0]) == 0  # read and cleared
    assert not sched.has_unfinished() and not sched.finished
    assert llm.cache.num_free_pages == llm.cache.num_pages
    llm.cache.check()
    # the engine serves again afterwards
    outs = llm.generate(prompts, SamplingParams(max_new_tokens=8))
    assert [o.token_ids for o in outs] == [plain_tokens(plain, p, 8) for p in prompts]
    # and the same with steps running ahead of the host
    ahead(llm)
    ids = [sched.add_request(p, SamplingParams(max_new_tokens=8)) for p in prompts]
    while sched._ahead is None:
        sched.step()
    flag[0] = 1
    with pytest.raises(ops.KernelError):
        sched.step()
    assert not sched.has_unfinished() and llm.cache.num_free_pages == llm.cache.num_pages


def test_admission_speaks_for_the_pages_of_the_whole_prompt(model_folder, plain_ops_engine):
    """Prompts are fed in portions, but a request is admitted only if the pages of ALL it has to feed are there beside
    what the running requests still need (the reference admits whole prompts: engine.py:220-225).  Three prompts of 40
    tokens (10 pages each) over 24 pages: two run, the third waits for one of them to end; nobody is put back.  Admitted
    by its first portion alone, the third would take pages that the others need and all three would be computed again
    and again."""
    llm, plain = make(model_folder, block_size=4, num_blocks=24, max_batch_size=3, max_num_batched_tokens=16, chunk_size=8)
    sched = llm.scheduler
    prompts = tiny_configs.seeded_tokens(256, [40, 40, 40], 21)
    ids = [sched.add_request(p, SamplingParams(max_new_tokens=4)) for p in prompts]
    most_running = 0
    while sched.has_unfinished():
        sched.step()
        most_running = max(most_running, len(sched.running))
    assert most_running == 2 and sched.stats.preemptions == 0
    for rid, prompt in zip(ids, prompts):
        assert sched.finished[rid].generated == plain_tokens(plain, prompt, 4)
    assert llm.cache.num_free_pages == llm.cache.num_pages
