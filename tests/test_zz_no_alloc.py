"""The attention entry point that allocates nothing, called through its exported C symbol.

Some programs that embed the kernel library may not allocate device memory where they call it:
they gave all memory to a pool of their own, or they run where the allocator is locked, or
they are bindings from a language that can pass pointers but has no allocator to lend.  For
them ``llm_attention_mma_static_scratch`` keeps the split-key attention's scratch memory in a
fixed array inside the library.  This test calls that symbol directly (ctypes, raw pointers,
the current stream), twice in a row on different inputs — the second call meets whatever the
first left in the shared array — and checks each result against the usual entry point's, which
gets its scratch memory from the caller.  It also checks that sizes beyond the array are
refused with a message instead of being run.

The file is named so that it is collected last: a run that stops at the first failure has then
already run every other test.
"""

from __future__ import annotations

import ctypes
from types import SimpleNamespace

import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOO_LARGE = 10003


def _library():
    from llmserve_triton_kernels_b200 import ops

    lib = ops.library()
    fn = lib.llm_attention_mma_static_scratch
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, i, vp, i, vp, vp, i, vp, vp, vp, i, i, i, i, i, i, i, f, i, i, i, i, vp]
    fn.restype = ctypes.c_int
    lib.llm_attention_static_scratch_error.restype = ctypes.c_char_p
    return ops, lib, fn


def _case(seed: int, requests: int, ctx_len: int, H: int, KV: int, D: int, page_size: int):
    g = torch.Generator().manual_seed(seed)
    pages_each = -(-ctx_len // page_size)
    pool = (torch.randn(requests * pages_each + 2, 2, KV, page_size, D, generator=g)).to(torch.bfloat16).to(DEV)
    table = torch.randperm(requests * pages_each, generator=g).to(torch.int32).view(requests, pages_each).to(DEV)
    q = torch.randn(requests, (H + 2 * KV) * D, generator=g).to(torch.bfloat16).to(DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    ctx = SimpleNamespace(
        cu_tokens=i32(list(range(requests + 1))), context_lens=i32([ctx_len - r for r in range(requests)]),
        token_request=i32(list(range(requests))), host_cu_tokens=list(range(requests + 1)), max_context_len=ctx_len,
    )
    return q, pool, table, ctx


def _call_static(fn, q, pool, table, ctx, H, KV, D, splits):
    n = q.shape[0]
    out = torch.zeros((n, H * D), dtype=torch.bfloat16, device=DEV)
    code = fn(
        q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), pool.data_ptr(), table.data_ptr(), table.shape[1],
        ctx.token_request.data_ptr(), ctx.cu_tokens.data_ptr(), ctx.context_lens.data_ptr(), n, n, H, KV, D,
        pool.shape[3], 0, float(D**-0.5), 0, 1, splits, 1, torch.cuda.current_stream().cuda_stream,
    )
    return code, out


def test_static_scratch_entry_point_matches_the_usual_one_twice_in_a_row():
    ops, lib, fn = _library()
    H, KV, D, page_size = 8, 2, 64, 16
    for seed, requests, ctx_len in ((1, 6, 900), (2, 3, 1500)):
        q, pool, table, ctx = _case(seed, requests, ctx_len, H, KV, D, page_size)
        want = ops.paged_attention(q, pool, table, ctx, num_heads=H, num_kv_heads=KV, head_dim=D, scale=D**-0.5)
        code, got = _call_static(fn, q, pool, table, ctx, H, KV, D, splits=6)
        assert code == 0, lib.llm_attention_static_scratch_error().decode()
        torch.cuda.synchronize()
        # the same kernel and the same split arithmetic: equal up to the order in which splits are merged
        torch.testing.assert_close(got.float(), want.float(), atol=1.6e-2, rtol=1.6e-2)
        assert got.float().abs().max() > 0
        # and both stand against the plain statement of the attention
        plain = plain_ops.paged_attention(q, pool, table, ctx, num_heads=H, num_kv_heads=KV, head_dim=D, scale=D**-0.5)
        torch.testing.assert_close(got.float(), plain.float(), atol=1.6e-2, rtol=1.6e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    _, lib, fn = _library()
    H, KV, D, page_size = 8, 2, 64, 16
    q, pool, table, ctx = _case(3, 4, 300, H, KV, D, page_size)
    n = q.shape[0]
    out = torch.zeros((n, H * D), dtype=torch.bfloat16, device=DEV)
    args = [q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), pool.data_ptr(), table.data_ptr(), table.shape[1],
            ctx.token_request.data_ptr(), ctx.cu_tokens.data_ptr(), ctx.context_lens.data_ptr(), n, n, H, KV, D,
            page_size, 0, float(D**-0.5), 0, 1, 4, 1, torch.cuda.current_stream().cuda_stream]
    too_many_rows = list(args)
    too_many_rows[11] = 16384  # n_tokens: times H times splits is far beyond the array
    assert fn(*too_many_rows) == TOO_LARGE
    assert b"exceeds the fixed scratch" in lib.llm_attention_static_scratch_error()
    big_head = list(args)
    big_head[14] = 256
    assert fn(*big_head) == TOO_LARGE
    assert b"head size" in lib.llm_attention_static_scratch_error()
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0  # nothing was launched
