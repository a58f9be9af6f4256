"""A plain torch statement of every device operation, with the signature of the engine's
``ops`` functions.  Two uses: the oracle of each kernel's own test on the GPU, and — patched
over ``ops`` by the ``plain_ops_engine`` fixture — a way to run the engine's host logic (batch
building, cache manager, step function, scheduler) on the CPU, where no kernel can run.
Everything is computed in float32 (float64 where noted) and rounded to the output type once.
"""

from __future__ import annotations

import torch

import plain_llama


def embed(ids, table):
    return table[ids.long()].float()


def rmsnorm(resid, weight, eps, delta=None, rows=None, out_dtype=torch.float32):
    if rows is not None:
        v = resid[rows.long()]
        if delta is not None:
            v = v + delta[rows.long()].float()
    else:
        if delta is not None:
            resid.add_(delta.float())
        v = resid
    y = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight
    return y.to(out_dtype)


def linear(x, w, out_dtype=None):
    out_dtype = out_dtype or x.dtype
    return (x.float() @ w.float().t()).to(out_dtype)


def _rotate(x, positions, table):
    """x [N, heads, D] float32, table [positions, D] = cos | sin halves."""
    half = x.shape[-1] // 2
    cs = table[positions.long()]
    cos, sin = cs[:, None, :half], cs[:, None, half:]
    a, b = x[..., :half], x[..., half:]
    return torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1)


def rope_kv_write(qkv, positions, table, slot_map, pool, num_heads, num_kv_heads, head_dim, write_kv=True):
    H, KV, D = num_heads, num_kv_heads, head_dim
    n = qkv.shape[0]
    q = qkv[:, : H * D].float().view(n, H, D)
    if table is not None:
        q = _rotate(q, positions, table)
    qkv[:, : H * D] = q.reshape(n, H * D).to(qkv.dtype)
    if not write_kv:
        return
    k = qkv[:, H * D : (H + KV) * D].float().view(n, KV, D)
    if table is not None:
        k = _rotate(k, positions, table)
    v = qkv[:, (H + KV) * D : (H + 2 * KV) * D].view(n, KV, D)
    page_size = pool.shape[3]
    page = (slot_map // page_size).long()
    off = (slot_map % page_size).long()
    pool[page, 0, :, off, :] = k.to(pool.dtype)
    pool[page, 1, :, off, :] = v.to(pool.dtype)


def rope_inplace(x, positions, table):
    x.copy_(_rotate(x.float(), positions, table).to(x.dtype))


def paged_attention(qkv, pool, page_table, ctx, *, num_heads, num_kv_heads, head_dim, scale, window=None):
    H, KV, D = num_heads, num_kv_heads, head_dim
    page_size = pool.shape[3]
    out = torch.empty((qkv.shape[0], H * D), dtype=qkv.dtype, device=qkv.device)
    cu = ctx.cu_tokens.tolist()
    lens = ctx.context_lens.tolist()
    for r in range(len(lens)):
        t0, t1, n = cu[r], cu[r + 1], lens[r]
        pages = page_table[r, : -(-n // page_size)].long()
        k = pool[pages, 0].float().permute(1, 0, 2, 3).reshape(KV, -1, D)[:, :n]
        v = pool[pages, 1].float().permute(1, 0, 2, 3).reshape(KV, -1, D)[:, :n]
        q = qkv[t0:t1, : H * D].float().view(t1 - t0, H, D).transpose(0, 1)
        k = k.repeat_interleave(H // KV, dim=0)
        v = v.repeat_interleave(H // KV, dim=0)
        s = torch.einsum("htd,hsd->hts", q, k) * scale
        pos = torch.arange(n - (t1 - t0), n, device=qkv.device)[:, None]
        j = torch.arange(n, device=qkv.device)[None, :]
        visible = j <= pos
        if window:
            visible = visible & (j > pos - window)
        s = s.masked_fill(~visible[None], float("-inf"))
        o = torch.einsum("hts,hsd->htd", torch.softmax(s, dim=-1), v)
        out[t0:t1] = o.transpose(0, 1).reshape(t1 - t0, H * D).to(out.dtype)
    return out


def swiglu(gate_up):
    inter = gate_up.shape[1] // 2
    g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    return (g * torch.sigmoid(g) * u).to(gate_up.dtype)


def add_bias(x, bias):
    x.copy_((x.float() + bias.float()).to(x.dtype))
    return x


def linear_swiglu(x, w_gate_up):
    return swiglu(linear(x, w_gate_up))


def linear_qkv_rope(*args, **kwargs):
    return None  # "not taken": the caller runs the product, the rotation and the write one by one


def argmax(logits):
    return torch.argmax(logits, dim=-1).to(torch.int32)


def sample(logits, temperature, top_k, top_p, seeds, counters):
    out = []
    for r in range(logits.shape[0]):
        u = plain_llama.uniform_from(int(seeds[r]) & ((1 << 64) - 1), int(counters[r]))
        out.append(
            plain_llama.sample_token(logits[r].cpu(), float(temperature[r]), int(top_k[r]), float(top_p[r]), u)
        )
    return torch.tensor(out, dtype=torch.int32, device=logits.device)


ALL = (
    "embed",
    "rmsnorm",
    "linear",
    "rope_kv_write",
    "rope_inplace",
    "paged_attention",
    "swiglu",
    "add_bias",
    "linear_swiglu",
    "linear_qkv_rope",
    "argmax",
    "sample",
)
