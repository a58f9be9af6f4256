"""A plain, slow implementation of the Llama decoder: whole sequences, no cache, one function per
part, written from the reference's formulas.  It shares no code with the engine: it reads
config.json and the safetensors file itself and uses only elementary torch operations.

It was compared once with the reference's own model code on the CPU (tiny random models, see
``tests/golden/make_golden.py``); ``tests/test_plain.py`` re-checks it against those stored
outputs.

``window`` and ``schedule`` are not Llama's: they exist so that the engine's general parts
(windowed attention, an order of layers that repeats one or shares a cache) can be checked
against the same plain arithmetic.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def read_model(model_dir) -> tuple[dict, dict[str, torch.Tensor]]:
    """config.json as a dict and every tensor as float32."""
    from safetensors import safe_open

    path = Path(model_dir)
    cfg = json.loads((path / "config.json").read_text())
    weights = {}
    for f in sorted(path.glob("*.safetensors")):
        with safe_open(str(f), framework="pt", device="cpu") as sf:
            for k in sf.keys():
                weights[k] = sf.get_tensor(k).to(torch.float32)
    return cfg, weights


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """src/llmserve/model/llama.py:24-28: x * rsqrt(mean(x^2) + eps) * weight, in 32-bit."""
    x = x.float()
    return weight * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float):
    """src/llmserve/model/llama.py:31-39: inv_freq = 1 / theta^(2i/D); angle = p * inv_freq; the
    angles are repeated for the two halves of the head."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = 1.0 / (theta**exponent)
    freqs = positions.float()[..., None] * inv_freq
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """src/llmserve/model/llama.py:42-44."""
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """src/llmserve/model/llama.py:47-54, for x [heads, T, D] and cos/sin [T, D]."""
    return x * cos[None] + rotate_half(x) * sin[None]


def attention_scores(q, k, v, scale: float, window: int | None = None) -> torch.Tensor:
    """Causal softmax attention for one sequence: q [H, T, D], k/v [KV, T, D] -> [H, T, D].
    Consecutive query heads share a key/value head (src/llmserve/model/llama.py:94-97,
    repeat_interleave); key j is visible to query i iff j <= i
    (src/llmserve/kvcache/paged.py:106-109) and, with a window, j > i - window; the scale is
    1/sqrt(D) in the reference (the default of scaled_dot_product_attention,
    src/llmserve/kvcache/paged.py:110)."""
    H, T, D = q.shape
    rep = H // k.shape[0]
    k = k.repeat_interleave(rep, dim=0)
    v = v.repeat_interleave(rep, dim=0)
    s = torch.einsum("htd,hsd->hts", q, k) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & (j > i - window)
    s = s.masked_fill(~visible[None], float("-inf"))
    return torch.einsum("hts,hsd->htd", torch.softmax(s, dim=-1), v)


def attention_layer(x, w, prefix, cfg, window=None, shared_kv=None):
    """src/llmserve/model/llama.py:78-88: projections, rotary on q and k, attention, output
    projection.  Returns the layer's contribution and its (rotated k, v) so that another layer
    can share them.  Bias vectors are added where ``w`` holds them: the reference's q, k and v
    projections take one as an option (src/llmserve/model/llama.py:64-66), its output projection
    never does (an ``o_proj.bias`` here serves the engine's general part only)."""
    T = x.shape[0]
    H, KV = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    D = cfg["hidden_size"] // H
    theta = float(cfg.get("rope_theta", 10000.0))
    cos, sin = rope_cos_sin(torch.arange(T), D, theta)
    def project(name):
        y = x @ w[prefix + name + ".weight"].T
        return y + w[prefix + name + ".bias"] if prefix + name + ".bias" in w else y

    q = project("q_proj").view(T, H, D).transpose(0, 1)
    q = apply_rope(q, cos, sin)
    if shared_kv is None:
        k = project("k_proj").view(T, KV, D).transpose(0, 1)
        v = project("v_proj").view(T, KV, D).transpose(0, 1)
        k = apply_rope(k, cos, sin)
    else:
        k, v = shared_kv
    o = attention_scores(q, k, v, 1.0 / math.sqrt(D), window)
    x = o.transpose(0, 1).reshape(T, H * D)
    return project("o_proj"), (k, v)


def swiglu_mlp(x, w, prefix):
    """src/llmserve/model/llama.py:119-120: down(silu(gate(x)) * up(x)), silu(z) = z * sigmoid(z).  The reference's
    three products carry no bias; vectors ``*_proj.bias`` in ``w`` are added for the engine's general part."""
    def project(x, name):
        y = x @ w[prefix + name + ".weight"].T
        return y + w[prefix + name + ".bias"] if prefix + name + ".bias" in w else y

    g, u = project(x, "gate_proj"), project(x, "up_proj")
    return project((g * torch.sigmoid(g)) * u, "down_proj")


def forward(cfg: dict, w: dict[str, torch.Tensor], tokens, windows=None, schedule=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (src/llmserve/model/llama.py:155-185 and 131-135:
    embedding; per layer x += attn(norm(x)), x += mlp(norm(x)); final norm; output matrix, which
    is the token table when tie_word_embeddings).

    ``windows``: per layer a window or None.  ``schedule``: list of (layer, cache_of) — the layer
    whose weights run, and the index of an earlier entry whose keys and values it reads."""
    eps = float(cfg.get("rms_norm_eps", 1e-5))
    L = cfg["num_hidden_layers"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["model.embed_tokens.weight"][tokens]
    schedule = schedule or [(i, None) for i in range(L)]
    kept = []
    for layer, cache_of in schedule:
        p = f"model.layers.{layer}."
        window = None if windows is None else windows[layer]
        h = rms_norm(x, w[p + "input_layernorm.weight"], eps)
        shared = None if cache_of is None else kept[cache_of]
        a, kv = attention_layer(h, w, p + "self_attn.", cfg, window, shared)
        kept.append(kv)
        x = x + a
        x = x + swiglu_mlp(rms_norm(x, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")
    x = rms_norm(x, w["model.norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return x @ head.T


# ------------------------------------------------------------------------------------------------
# sampling
# ------------------------------------------------------------------------------------------------
_MASK = (1 << 64) - 1


def uniform_from(seed: int, counter: int) -> float:
    """The engine's counter-based uniform number in [0, 1): a 64-bit mix of (seed, counter), top
    24 bits.  The reference draws with torch.multinomial from a per-request generator
    (src/llmserve/sampling/sampler.py:8-13, 38-39), whose stream no kernel can reproduce; the
    distribution is the same."""
    x = (seed ^ ((counter * 0x9E3779B97F4A7C15 + 0xD1B54A32D192ED03) & _MASK)) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    x = x ^ (x >> 31)
    return (x >> 40) / 16777216.0


def filtered_probs(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
    """src/llmserve/sampling/sampler.py:23-38: divide by the temperature; keep values >= the k-th
    largest; sort descending and drop a token if the mass before it exceeds top_p; softmax."""
    x = logits.float() / temperature
    if top_k > 0:
        k = min(top_k, x.numel())
        kth = torch.topk(x, k).values[-1]
        x = x.masked_fill(x < kth, float("-inf"))
    if top_p < 1.0:
        sorted_x, idx = torch.sort(x, descending=True)
        probs = torch.softmax(sorted_x, dim=-1)
        remove = (probs.cumsum(-1) - probs) > top_p
        sorted_x = sorted_x.masked_fill(remove, float("-inf"))
        x = torch.full_like(x, float("-inf")).scatter(-1, idx, sorted_x)
    return torch.softmax(x, dim=-1)


def sample_token(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """Greedy when temperature <= 0 (src/llmserve/sampling/sampler.py:20-21); else the first token
    in vocabulary order whose cumulative probability exceeds u."""
    if temperature <= 0:
        return int(torch.argmax(logits))
    cdf = filtered_probs(logits, temperature, top_k, top_p).double().cumsum(-1)
    return int(min(int(torch.searchsorted(cdf, torch.tensor(u * float(cdf[-1]), dtype=torch.float64), right=True)), logits.numel() - 1))


def generate(cfg, w, prompt, max_new_tokens, temperature=0.0, top_k=0, top_p=1.0, seed=0, eos=None, **kw):
    """No cache: the whole sequence is recomputed for every token
    (src/llmserve/baseline/naive.py:20-56).  The n-th drawn token uses counter n."""
    tokens = list(prompt)
    out = []
    for n in range(max_new_tokens):
        logits = forward(cfg, w, tokens, **kw)[-1]
        tok = sample_token(logits, temperature, top_k, top_p, uniform_from(seed, n))
        out.append(tok)
        tokens.append(tok)
        if eos is not None and tok == eos:
            break
    return out
