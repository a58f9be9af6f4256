"""Checked mode: a step's integer arrays are looked over on the device before the kernels that index with them.

The check kernels only read (and repair) the step's own small arrays, never the cache or a weight, so a test may hand
them a wrong index without any memory being touched out of bounds.  The engine-level case plants a slot that lies INSIDE
the pool but is not the one the page table gives: whatever the check did with it, no access could leave the pool.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_llama
import tiny_configs

pytestmark = pytest.mark.gpu


def _context(counts, starts, vocab=100, seed=0):
    from llmserve_triton_kernels_b200.engine.batch import StepContext

    dev = torch.device("cuda:0")
    n, r = sum(counts), len(counts)
    cu = np.zeros(r + 1, dtype=np.int32)
    cu[1:] = np.cumsum(counts)
    g = np.random.default_rng(seed)
    t = lambda a: torch.tensor(np.asarray(a, dtype=np.int32), device=dev)
    positions = np.concatenate([np.arange(s, s + c) for s, c in zip(starts, counts)])
    return StepContext(
        num_tokens=n, num_requests=r, num_logits=r, token_ids=t(g.integers(0, vocab, n)), positions=t(positions),
        token_request=t(np.repeat(np.arange(r), counts)), cu_tokens=t(cu), context_lens=t([s + c for s, c in zip(starts, counts)]),
        logit_rows=t(cu[1:] - 1), state_slots=t(np.arange(r)), host_cu_tokens=cu.tolist(), host_context_lens=None,
        host_state_slots=None, max_query_len=max(counts), max_context_len=max(s + c for s, c in zip(starts, counts)),
    )


def _tables(counts, starts, page_size, num_pages, seed=1):
    """A page table that gives every request pages of its own, in a shuffled order, and the slots that follow from it."""
    dev = torch.device("cuda:0")
    pages = [-(-(s + c) // page_size) for s, c in zip(starts, counts)]
    order = np.random.default_rng(seed).permutation(num_pages)[: sum(pages)]
    table = np.zeros((len(counts), max(pages)), dtype=np.int32)
    at = 0
    for r, p in enumerate(pages):
        table[r, :p] = order[at : at + p]
        at += p
    slots = []
    for r, (s, c) in enumerate(zip(starts, counts)):
        pos = np.arange(s, s + c)
        slots.append(table[r, pos // page_size] * page_size + pos % page_size)
    return torch.tensor(table, device=dev), torch.tensor(np.concatenate(slots).astype(np.int32), device=dev)


COUNTS, STARTS, PAGE, PAGES = [5, 1, 19, 2], [0, 37, 8, 15], 8, 40


def _run(ctx, table, slots, window=None):
    from llmserve_triton_kernels_b200 import ops

    ops.check_step_arrays(ctx, 100, 64, 4)
    ops.check_page_group(ctx, table, slots, PAGE, PAGES, window, 0)
    torch.cuda.synchronize()
    ops.check_device_errors()


def test_sound_arrays_pass():
    ctx = _context(COUNTS, STARTS)
    table, slots = _tables(COUNTS, STARTS, PAGE, PAGES)
    before = (table.clone(), slots.clone(), ctx.token_ids.clone())
    _run(ctx, table, slots)
    assert torch.equal(table, before[0]) and torch.equal(slots, before[1]) and torch.equal(ctx.token_ids, before[2])


@pytest.mark.parametrize("what,message", [
    ("token", "a token id outside the vocabulary"), ("position", "a position beyond"), ("owner", "a request it does not belong to"),
    ("length", "a context length"), ("row", "a wanted row"), ("state", "a state slot"), ("page", "a page table entry outside the pool"),
    ("negative page", "a page table entry outside the pool"), ("slot", "a slot that is outside the pool or disagrees"),
    ("far slot", "a slot that is outside the pool or disagrees"),
])
def test_each_wrong_index_is_named_and_replaced(what, message):
    from llmserve_triton_kernels_b200 import ops

    ctx = _context(COUNTS, STARTS)
    table, slots = _tables(COUNTS, STARTS, PAGE, PAGES)
    if what == "token":
        ctx.token_ids[7] = 100
    elif what == "position":
        ctx.positions[3] = 64
    elif what == "owner":
        ctx.token_request[6] = 3
    elif what == "length":
        ctx.context_lens[2] = 5
    elif what == "row":
        ctx.logit_rows[1] = 27
    elif what == "state":
        ctx.state_slots[3] = 4
    elif what == "page":
        table[2, 1] = PAGES
    elif what == "negative page":
        table[1, 4] = -1
    elif what == "slot":
        slots[9] = int(slots[9]) ^ 1
    elif what == "far slot":
        slots[0] = PAGES * PAGE
    with pytest.raises(ops.KernelError, match=message) as err:
        _run(ctx, table, slots)
    assert "checked mode" in str(err.value)
    # what the kernels after the check would have read is inside its bounds again
    assert int(ctx.token_ids.max()) < 100 and int(ctx.positions.max()) < 64 and int(ctx.logit_rows.max()) < sum(COUNTS)
    assert int(ctx.state_slots.max()) < 4 and 0 <= int(slots.min()) and int(slots.max()) < PAGES * PAGE
    live = [(r, p) for r, (s, c) in enumerate(zip(STARTS, COUNTS)) for p in range(-(-(s + c) // PAGE))]
    assert all(0 <= int(table[r, p]) < PAGES for r, p in live)
    if what != "owner":  # (an owner that is merely another request of the step is named, not replaced)
        _run(ctx, table, slots)  # the record is clear again and the repaired arrays pass


def test_pages_that_a_window_has_passed_are_not_looked_at():
    from llmserve_triton_kernels_b200 import ops

    ctx = _context([1], [50])
    table, slots = _tables([1], [50], PAGE, PAGES)
    table[0, :4] = -1  # keys 0..31: a window of 16 has long passed them
    _run(ctx, table, slots, window=16)
    with pytest.raises(ops.KernelError, match="a page table entry outside the pool"):
        _run(ctx, table, slots, window=None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_checked_engine_gives_the_same_logits_and_a_wrong_slot_stops_it(dtype, model_folder, monkeypatch):
    from llmserve_triton_kernels_b200 import LLM, ops
    from llmserve_triton_kernels_b200.engine.batch import StepEntry

    cfg = tiny_configs.TINY_B
    folder = model_folder(cfg, 2, torch.float32 if dtype == "float32" else torch.bfloat16)
    plain_cfg, w = plain_llama.read_model(folder)
    seqs = tiny_configs.seeded_tokens(cfg["vocab_size"], [41, 23, 30], 77)
    refs = [plain_llama.forward(plain_cfg, w, s) for s in seqs]
    monkeypatch.setattr(ops, "_checked", True)
    llm = LLM(folder, dtype=dtype, device="cuda:0", block_size=8, num_blocks=14, max_batch_size=4, max_num_batched_tokens=64)
    step = llm.step_function
    before = ops.launch_count()
    step([StepEntry("a", seqs[0][:30], []), StepEntry("b", seqs[1][:9], [8])])
    assert ops.launch_count() - before >= 2  # the check kernels ran with the step
    rtol = 2e-5 if dtype == "float32" else 2e-2
    for k in range(3):  # decode steps: captured with the checks inside
        logits = step([StepEntry("a", [seqs[0][30 + k]], [0]), StepEntry("b", [seqs[1][9 + k]], [0])]).float().cpu()
        for row, (r, at) in enumerate([(0, 30 + k), (1, 9 + k)]):
            ref = refs[r][at]
            assert float((logits[row] - ref).abs().max()) <= rtol * float(ref.abs().max())
    torch.cuda.synchronize()
    ops.check_device_errors()
    # a slot inside the pool that is not the one the page table gives: the step's arrays as the cache manager makes them,
    # with one slot moved to its neighbour
    real = step.cache.step_tables

    def wrong(pairs):
        groups, state = real(pairs)
        table, slots = groups[0]
        slots = slots.copy()
        slots[1] ^= 1
        return [(table, slots)] + list(groups[1:]), state

    monkeypatch.setattr(step.cache, "step_tables", wrong)
    step([StepEntry("c", seqs[2][:12], [11])])
    torch.cuda.synchronize()
    with pytest.raises(ops.KernelError, match="disagrees with the page table"):
        ops.check_device_errors()
