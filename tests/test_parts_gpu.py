"""Each part alone against the plain implementation, and the generality of the assembly: a toy
mixer with state of its own, a windowed layer, a layer that runs twice and a layer that reads
another layer's cache — registered, built and stepped from the test alone, without a change to
the framework's files."""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass

import pytest
import torch
from safetensors.torch import save_file

import plain_llama
import tiny_configs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, std=1.0, dtype=torch.float32):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * std).to(dtype)


# ------------------------------------------------------------------ parts alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from llmserve_triton_kernels_b200.parts import PartSpec, build_part

    norm = build_part("norm", PartSpec("rms_norm", {"size": 72, "eps": 1e-3}))
    assert list(norm.tensors()) == ["weight"] and norm.tensors()["weight"].shape == (72,)
    w = 1 + rnd(72, seed=1, std=0.1)
    norm.bind({"weight": w.to(torch.bfloat16 if dtype == torch.bfloat16 else torch.float32)}, dtype, DEV)
    x, d = rnd(5, 72, seed=2), rnd(5, 72, seed=3).to(dtype)
    resid = x.to(DEV)
    got = norm.add_forward(resid, d.to(DEV))
    w_used = w.to(torch.bfloat16).float() if dtype == torch.bfloat16 else w
    want = plain_llama.rms_norm(x + d.float(), w_used, 1e-3)
    tol = 2e-6 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(got.float().cpu(), want, atol=tol, rtol=tol)
    torch.testing.assert_close(resid.cpu(), x + d.float(), atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotary_part(dtype):
    from llmserve_triton_kernels_b200.parts import PartSpec, build_part

    rot = build_part("position", PartSpec("rotary", {"head_dim": 48, "theta": 777.0, "max_positions": 90}))
    rot.bind({}, dtype, DEV)
    positions = torch.tensor([0, 1, 89, 33, 7], dtype=torch.int32, device=DEV)
    q, k = rnd(5, 3, 48, seed=4).to(dtype), rnd(5, 1, 48, seed=5).to(dtype)
    qd, kd = q.to(DEV), k.to(DEV)
    rot.apply(qd, kd, positions)
    cos, sin = plain_llama.rope_cos_sin(positions.cpu(), 48, 777.0)
    tol = 2e-6 if dtype == torch.float32 else 2e-2
    for got, x in ((qd, q), (kd, k)):
        want = plain_llama.apply_rope(x.float().transpose(0, 1), cos, sin).transpose(0, 1)
        torch.testing.assert_close(got.float().cpu(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype, bias):
    from llmserve_triton_kernels_b200.parts import PartSpec, build_part

    ff = build_part("feed_forward", PartSpec("gated_mlp", {"hidden_size": 40, "intermediate_size": 104, "bias": bias}))
    w = {"gate_proj.weight": rnd(104, 40, seed=6, std=0.2), "up_proj.weight": rnd(104, 40, seed=7, std=0.2),
         "down_proj.weight": rnd(40, 104, seed=8, std=0.2)}
    if bias:
        w.update({"gate_proj.bias": rnd(104, seed=60), "up_proj.bias": rnd(104, seed=61), "down_proj.bias": rnd(40, seed=62)})
    w = {k: v.to(dtype) for k, v in w.items()}
    assert {k: v.shape for k, v in ff.tensors().items()} == {k: tuple(v.shape) for k, v in w.items()}
    ff.bind(w, dtype, DEV)
    for n in (3, 70):  # few rows: the fused decode kernels in bfloat16; many: the library product
        x = rnd(n, 40, seed=9).to(dtype)
        got = ff.forward(x.to(DEV), None)
        want = plain_llama.swiglu_mlp(x.float(), {"p." + k: v.float() for k, v in w.items()}, "p.")
        tol = 1e-5 if dtype == torch.float32 else 3e-2
        torch.testing.assert_close(got.float().cpu(), want, atol=tol * float(want.abs().max()), rtol=tol)
    with pytest.raises(ValueError, match="activation"):
        build_part("feed_forward", PartSpec("gated_mlp", {"hidden_size": 8, "intermediate_size": 8, "activation": "relu"}))


def _attention_alone(dtype, window, page_size, D=32, bias=False, position_kind="rotary"):
    """The attention part over a cache of its own, fed in three portions, against the plain layer."""
    from llmserve_triton_kernels_b200.cache import CacheManager
    from llmserve_triton_kernels_b200.engine.batch import StepEntry, pack_step
    from llmserve_triton_kernels_b200.models.plan import LayerRun
    from llmserve_triton_kernels_b200.parts import PartSpec, build_part

    H, KV, hidden, T = 6, 2, 80, 37
    cfg = {"num_attention_heads": H, "num_key_value_heads": KV, "hidden_size": H * D, "rope_theta": 3000.0}
    rotary = PartSpec(position_kind, {"head_dim": D, "theta": 3000.0, "max_positions": 64})
    attn = build_part("mixer", PartSpec("attention", {
        "hidden_size": hidden, "num_heads": H, "num_kv_heads": KV, "head_dim": D, "scale": D**-0.5, "window": window,
        "position": rotary, "qkv_bias": bias, "out_bias": bias}))
    w = {"q_proj.weight": rnd(H * D, hidden, seed=10, std=0.1), "k_proj.weight": rnd(KV * D, hidden, seed=11, std=0.1),
         "v_proj.weight": rnd(KV * D, hidden, seed=12, std=0.1), "o_proj.weight": rnd(hidden, H * D, seed=13, std=0.1)}
    if bias:
        w.update({"q_proj.bias": rnd(H * D, seed=70), "k_proj.bias": rnd(KV * D, seed=71), "v_proj.bias": rnd(KV * D, seed=72),
                  "o_proj.bias": rnd(hidden, seed=73)})
    w = {k: v.to(dtype) for k, v in w.items()}
    assert {k: v.shape for k, v in attn.tensors().items()} == {k: tuple(v.shape) for k, v in w.items()}
    attn.bind(w, dtype, DEV)
    cache = CacheManager([attn.cache_spec()], [LayerRun(0)], page_size=page_size, num_pages=16, max_requests=2, dtype=dtype, device=DEV)
    x = rnd(T, hidden, seed=14).to(dtype)
    cache.add_request("r")
    outs, fed = [], 0
    for n in (20, 1, 16):
        entries = [StepEntry("r", [0] * n, [])]
        cache.reserve([("r", n)])
        arrays, slots = cache.step_tables([("r", n)])
        ctx, group_tensors, _ = pack_step(entries, [fed], slots, arrays, DEV)
        view = cache.views(group_tensors, ctx.state_slots, ctx.host_state_slots)[0]
        outs.append(attn.forward(x[fed : fed + n].to(DEV), ctx, view))
        cache.commit([("r", n)])
        fed += n
    got = torch.cat(outs).float().cpu()
    # the plain layer takes hidden-size inputs through the same projections
    plain_w = {"p." + k: v.float() for k, v in w.items()}
    plain_cfg = dict(cfg)
    plain_cfg["hidden_size"] = H * D  # head_dim is derived from it there
    want, _ = plain_llama.attention_layer(x.float(), plain_w, "p.", plain_cfg, window)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    torch.testing.assert_close(got, want, atol=tol * float(want.abs().max()), rtol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,page_size", [(None, 8), (5, 4), (16, 16)])
def test_attention_part(dtype, window, page_size):
    _attention_alone(dtype, window, page_size)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [20, 100, 64])
def test_attention_part_at_head_sizes_that_are_no_multiple_of_16_and_with_biases(dtype, D):
    """Head sizes 20 and 100 (a hidden size of 3200 over 32 heads) take the general attention kernel in both
    precisions; with ``qkv_bias`` and ``out_bias`` the projections carry bias vectors, and the fused decode kernels
    (which have no place for one) stand aside for the product and a bias kernel."""
    _attention_alone(dtype, None, 8, D=D)
    _attention_alone(dtype, 9, 16, D=D, bias=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_rotary_table_of_another_layout_is_not_taken_for_the_half_rotation(dtype):
    """A position encoding that tabulates its angles like the rotary one but says nothing of how lanes pair
    (``rotary_layout`` None) must be asked to ``apply`` itself: the kernels that rotate while they store keys know the
    half-rotation layout only.  Here the encoding's own ``apply`` IS the half rotation, so the plain layer stays the
    oracle; a call counter shows which way was taken."""
    from llmserve_triton_kernels_b200.parts import register_part
    from llmserve_triton_kernels_b200.parts.rotary import RotaryEmbedding

    calls = []

    class OtherLayout(RotaryEmbedding):
        rotary_layout = None

        def apply(self, q, k, positions):
            calls.append(q.shape[0])
            super().apply(q, k, positions)

    register_part("position", "other_layout_rotary", OtherLayout)
    _attention_alone(dtype, None, 8, position_kind="other_layout_rotary")
    assert calls == [20, 1, 16]


# ------------------------------------------------------------------ a toy architecture, defined here
@dataclass(frozen=True)
class ToyConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_heads: int
    num_kv_heads: int
    window: int
    decay: float
    eps: float
    max_positions: int
    architecture = "ToyForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: d[k] for k in cls.__dataclass_fields__})

    def to_dict(self):
        return {**asdict(self), "architectures": [self.architecture]}


def register_toy():
    """A mixer that keeps a running mean per request (state of fixed size), and an architecture
    whose order runs: attention; the toy mixer; windowed attention; layer 0 again (a second cache
    of its own); and a layer without key/value projections that reads entry 0's cache."""
    from llmserve_triton_kernels_b200.config import register_architecture
    from llmserve_triton_kernels_b200.models.plan import LayerRun, LayerSpec, ModelPlan
    from llmserve_triton_kernels_b200.parts import Mixer, PartSpec, StateSpec, TensorSpec, register_part

    class RunningMeanMixer(Mixer):
        def __init__(self, hidden_size: int, decay: float):
            self.hidden_size, self.decay = hidden_size, decay

        def tensors(self):
            return {"mix.weight": TensorSpec((self.hidden_size, self.hidden_size))}

        def bind(self, tensors, dtype, device):
            self.w = tensors["mix.weight"].to(device=device, dtype=torch.float32)
            self.dtype = dtype

        def cache_spec(self):
            return StateSpec((self.hidden_size,), torch.float32)

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x, dtype=torch.float32)
            cu = ctx.host_cu_tokens
            for r, slot in enumerate(cache.host_slots):  # the tokens of a request, in order
                s = cache.states[slot]
                for t in range(cu[r], cu[r + 1]):
                    s = self.decay * s + (1 - self.decay) * x[t].float()
                    out[t] = s
                cache.states[slot] = s
            return (out @ self.w.t()).to(self.dtype)

    register_part("mixer", "running_mean", RunningMeanMixer)

    def plan(cfg: ToyConfig) -> ModelPlan:
        D = cfg.hidden_size // cfg.num_heads
        norm = {"size": cfg.hidden_size, "eps": cfg.eps}
        rotary = PartSpec("rotary", {"head_dim": D, "theta": 10000.0, "max_positions": cfg.max_positions})

        def attention(i, window=None, own_kv=True):
            return PartSpec("attention", {"hidden_size": cfg.hidden_size, "num_heads": cfg.num_heads,
                                          "num_kv_heads": cfg.num_kv_heads, "head_dim": D, "scale": D**-0.5, "window": window,
                                          "position": rotary, "own_kv": own_kv}, f"model.layers.{i}.self_attn.")

        def layer(i, mixer):
            p = f"model.layers.{i}."
            return LayerSpec(PartSpec("pre_norm"), mixer_norm=PartSpec("rms_norm", norm, p + "input_layernorm."), mixer=mixer,
                             ff_norm=PartSpec("rms_norm", norm, p + "post_attention_layernorm."),
                             feed_forward=PartSpec("gated_mlp", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size}, p + "mlp."))

        layers = (layer(0, attention(0)), layer(1, PartSpec("running_mean", {"hidden_size": cfg.hidden_size, "decay": cfg.decay}, "model.layers.1.toy.")),
                  layer(2, attention(2, window=cfg.window)), layer(3, attention(3, own_kv=False)))
        schedule = (LayerRun(0), LayerRun(1), LayerRun(2), LayerRun(0), LayerRun(3, cache_of=0))
        return ModelPlan(cfg.hidden_size, cfg.vocab_size, cfg.max_positions, "model.embed_tokens.weight", layers, schedule,
                         PartSpec("rms_norm", norm, "model.norm."), "lm_head.weight")

    register_architecture("ToyForCausalLM", ToyConfig, plan)


def toy_plain_forward(cfg: ToyConfig, w, tokens):
    """The toy model on a whole sequence, in plain torch (the Llama parts are plain_llama's)."""
    lcfg = {"num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads, "hidden_size": cfg.hidden_size,
            "rope_theta": 10000.0}
    x = w["model.embed_tokens.weight"][torch.as_tensor(tokens)]
    kept = {}
    for entry, (layer, cache_of) in enumerate([(0, None), (1, None), (2, None), (0, None), (3, 0)]):
        p = f"model.layers.{layer}."
        h = plain_llama.rms_norm(x, w[p + "input_layernorm.weight"], cfg.eps)
        if layer == 1:
            s, rows = torch.zeros(cfg.hidden_size), []
            for t in range(h.shape[0]):
                s = cfg.decay * s + (1 - cfg.decay) * h[t]
                rows.append(s)
            a = torch.stack(rows) @ w[p + "toy.mix.weight"].T
        else:
            a, kv = plain_llama.attention_layer(h, w, p + "self_attn.", lcfg, cfg.window if layer == 2 else None,
                                                None if cache_of is None else kept[cache_of])
            kept[entry] = kv
        x = x + a
        x = x + plain_llama.swiglu_mlp(plain_llama.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.eps), w, p + "mlp.")
    return plain_llama.rms_norm(x, w["model.norm.weight"], cfg.eps) @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype,storage,rtol", [("float32", torch.float32, 3e-5), ("bfloat16", torch.bfloat16, 3e-2)])
def test_toy_architecture_with_a_stateful_mixer_is_registered_built_and_stepped(dtype, storage, rtol, tmp_path):
    from llmserve_triton_kernels_b200 import LLM, SamplingParams
    from llmserve_triton_kernels_b200.config import unregister_architecture
    from llmserve_triton_kernels_b200.engine.batch import StepEntry
    from llmserve_triton_kernels_b200.weights import write_random_model

    register_toy()
    try:
        cfg = ToyConfig(vocab_size=200, hidden_size=64, intermediate_size=88, num_heads=4, num_kv_heads=2, window=6,
                        decay=0.7, eps=1e-5, max_positions=96)
        folder = write_random_model(tmp_path, cfg, seed=3, std=0.05, dtype=storage)
        assert json.loads((folder / "config.json").read_text())["architectures"] == ["ToyForCausalLM"]
        _, w = plain_llama.read_model(folder)
        assert "model.layers.1.toy.mix.weight" in w and "model.layers.3.self_attn.k_proj.weight" not in w
        llm = LLM(folder, dtype=dtype, device=DEV, block_size=4, num_blocks=40, max_batch_size=3, max_num_batched_tokens=32, chunk_size=8)
        assert not llm.step_function.use_graphs  # the toy mixer walks requests on the host
        assert [g.spec.window for g in llm.cache.groups] == [None, 6]
        a, b = tiny_configs.seeded_tokens(200, [41, 23], 51)
        ref_a, ref_b = toy_plain_forward(cfg, w, a), toy_plain_forward(cfg, w, b)
        step = llm.step_function
        got_a, got_b = [], []
        # a in portions of changing size beside b's portions and single tokens
        ia = ib = 0
        for na, nb in ((7, 2), (2, 9), (16, 1), (1, 1), (5, 6), (10, 4)):
            entries = []
            if ia < len(a):
                entries.append(StepEntry("a", a[ia : ia + na], list(range(len(a[ia : ia + na])))))
            if ib < len(b):
                entries.append(StepEntry("b", b[ib : ib + nb], list(range(len(b[ib : ib + nb])))))
            out = step(entries).float().cpu()
            k = len(a[ia : ia + na]) if ia < len(a) else 0
            got_a.append(out[:k])
            got_b.append(out[k:])
            ia, ib = ia + na, ib + nb
        for got, ref in ((torch.cat(got_a), ref_a), (torch.cat(got_b), ref_b[: sum(x.shape[0] for x in got_b)])):
            assert float((got - ref[: got.shape[0]]).abs().max()) <= rtol * float(ref.abs().max())
        llm.cache.free_request("a")
        llm.cache.free_request("b")
        llm.cache.check()
        # and through the scheduler: greedy tokens of a fresh request equal the plain model's
        if dtype == "float32":
            out = llm.generate([a[:9]], SamplingParams(max_new_tokens=6))[0]
            tokens = list(a[:9])
            for _ in range(6):
                tokens.append(int(torch.argmax(toy_plain_forward(cfg, w, tokens)[-1])))
            assert out.token_ids == tokens[9:]
        assert llm.cache.num_free_pages == llm.cache.num_pages and llm.cache.slots.num_free == 3
    finally:
        unregister_architecture("ToyForCausalLM")


# ------------------------------------------------------------------ a second toy: routing, another position encoding, another norm
@dataclass(frozen=True)
class RoutedConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_heads: int
    num_kv_heads: int
    num_experts: int
    slope: float
    eps: float
    max_positions: int
    architecture = "RoutedToyForCausalLM"

    @classmethod
    def from_dict(cls, d):
        return cls(**{k: d[k] for k in cls.__dataclass_fields__})

    def to_dict(self):
        return {**asdict(self), "architectures": [self.architecture]}


def register_routed_toy():
    """Parts that the framework does not have, defined here: a feed-forward that routes every token to the one
    expert its 32-bit router prefers (gated by the router's softmax), a position encoding without a table (queries
    grow and keys shrink with the position, so that a score falls with the distance), and a norm that centres
    before it scales.  Layer 0 has a dense feed-forward and rotary positions, layer 1 the routed one and the toy
    positions: one model, different parts per layer."""
    from llmserve_triton_kernels_b200 import ops
    from llmserve_triton_kernels_b200.config import register_architecture
    from llmserve_triton_kernels_b200.models.plan import LayerRun, LayerSpec, ModelPlan
    from llmserve_triton_kernels_b200.parts import FeedForward, Norm, PartSpec, PositionEncoding, TensorSpec, register_part

    class RoutedExperts(FeedForward):
        def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int):
            self.h, self.i, self.e = hidden_size, intermediate_size, num_experts

        def tensors(self):
            specs = {"router.weight": TensorSpec((self.e, self.h))}
            for j in range(self.e):
                specs[f"experts.{j}.gate_up.weight"] = TensorSpec((2 * self.i, self.h))
                specs[f"experts.{j}.down.weight"] = TensorSpec((self.h, self.i))
            return specs

        def bind(self, tensors, dtype, device):
            self.router = tensors["router.weight"].to(device=device, dtype=torch.float32)  # router logits are 32-bit
            self.gate_up = [tensors[f"experts.{j}.gate_up.weight"].to(device=device, dtype=dtype).contiguous() for j in range(self.e)]
            self.down = [tensors[f"experts.{j}.down.weight"].to(device=device, dtype=dtype).contiguous() for j in range(self.e)]
            self.dtype = dtype

        def forward(self, x, ctx):
            probs = torch.softmax(x.float() @ self.router.t(), dim=-1)
            weight, choice = probs.max(dim=-1)
            out = torch.zeros((x.shape[0], self.h), dtype=torch.float32, device=x.device)
            for j in range(self.e):  # the framework's own kernels do an expert's products
                rows = torch.nonzero(choice == j).flatten()
                if rows.numel():
                    y = ops.linear(ops.linear_swiglu(x[rows].contiguous(), self.gate_up[j]), self.down[j], out_dtype=torch.float32)
                    out[rows] = y * weight[rows, None]
            return out.to(self.dtype)

    class DistanceDecay(PositionEncoding):
        def __init__(self, slope: float, max_positions: int):
            self.slope, self.max_positions = slope, max_positions

        def apply(self, q, k, positions):
            f = torch.exp(self.slope * positions.float() / self.max_positions)
            q.mul_(f[:, None, None].to(q.dtype))
            if k.shape[1]:
                k.mul_((1.0 / f)[:, None, None].to(k.dtype))

    class CentredNorm(Norm):
        def __init__(self, size: int, eps: float):
            self.size, self.eps = size, eps

        def tensors(self):
            return {"weight": TensorSpec((self.size,), init="ones_plus_normal")}

        def bind(self, tensors, dtype, device):
            self.weight = tensors["weight"].to(device=device, dtype=torch.float32)
            self.out_dtype = dtype

        def forward(self, x, rows=None):
            v = (x if rows is None else x[rows.long()]).float()
            v = v - v.mean(-1, keepdim=True)
            return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight).to(self.out_dtype)

    register_part("feed_forward", "routed_experts", RoutedExperts)
    register_part("position", "distance_decay", DistanceDecay)
    register_part("norm", "centred_norm", CentredNorm)

    def plan(cfg: RoutedConfig) -> ModelPlan:
        D = cfg.hidden_size // cfg.num_heads
        rms = {"size": cfg.hidden_size, "eps": cfg.eps}
        positions = (PartSpec("rotary", {"head_dim": D, "theta": 10000.0, "max_positions": cfg.max_positions}),
                     PartSpec("distance_decay", {"slope": cfg.slope, "max_positions": cfg.max_positions}))
        feed_forwards = (PartSpec("gated_mlp", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size}, "model.layers.0.mlp."),
                         PartSpec("routed_experts", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
                                                     "num_experts": cfg.num_experts}, "model.layers.1.moe."))
        layers = []
        for i in range(2):
            p = f"model.layers.{i}."
            attention = PartSpec("attention", {"hidden_size": cfg.hidden_size, "num_heads": cfg.num_heads, "num_kv_heads": cfg.num_kv_heads,
                                               "head_dim": D, "scale": D**-0.5, "position": positions[i]}, p + "self_attn.")
            ff_norm = PartSpec("rms_norm", rms, p + "post_attention_layernorm.") if i == 0 else PartSpec("centred_norm", rms, p + "ff_norm.")
            layers.append(LayerSpec(PartSpec("pre_norm"), mixer_norm=PartSpec("rms_norm", rms, p + "input_layernorm."), mixer=attention,
                                    ff_norm=ff_norm, feed_forward=feed_forwards[i]))
        return ModelPlan(cfg.hidden_size, cfg.vocab_size, cfg.max_positions, "model.embed_tokens.weight", tuple(layers),
                         (LayerRun(0), LayerRun(1)), PartSpec("rms_norm", rms, "model.norm."), "lm_head.weight")

    register_architecture("RoutedToyForCausalLM", RoutedConfig, plan)


def routed_plain_forward(cfg: RoutedConfig, w, tokens):
    """The routed toy on a whole sequence in plain torch; attention by plain_llama.attention_scores."""
    H, KV, D = cfg.num_heads, cfg.num_kv_heads, cfg.hidden_size // cfg.num_heads
    n = len(tokens)
    pos = torch.arange(n)
    x = w["model.embed_tokens.weight"][torch.as_tensor(tokens)]
    for i in range(2):
        p = f"model.layers.{i}."
        h = plain_llama.rms_norm(x, w[p + "input_layernorm.weight"], cfg.eps)
        q = (h @ w[p + "self_attn.q_proj.weight"].T).view(n, H, D).transpose(0, 1)
        k = (h @ w[p + "self_attn.k_proj.weight"].T).view(n, KV, D).transpose(0, 1)
        v = (h @ w[p + "self_attn.v_proj.weight"].T).view(n, KV, D).transpose(0, 1)
        if i == 0:
            cos, sin = plain_llama.rope_cos_sin(pos, D, 10000.0)
            q, k = plain_llama.apply_rope(q, cos, sin), plain_llama.apply_rope(k, cos, sin)
        else:
            f = torch.exp(cfg.slope * pos.float() / cfg.max_positions)[None, :, None]
            q, k = q * f, k / f
        a = plain_llama.attention_scores(q, k, v, D**-0.5)
        x = x + a.transpose(0, 1).reshape(n, H * D) @ w[p + "self_attn.o_proj.weight"].T
        if i == 0:
            x = x + plain_llama.swiglu_mlp(plain_llama.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.eps), w, p + "mlp.")
        else:
            c = x - x.mean(-1, keepdim=True)
            hn = c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + cfg.eps) * w[p + "ff_norm.weight"]
            probs = torch.softmax(hn @ w[p + "moe.router.weight"].T, dim=-1)
            weight, choice = probs.max(-1)
            y = torch.zeros_like(x)
            for t in range(n):
                j = int(choice[t])
                gu = hn[t] @ w[p + f"moe.experts.{j}.gate_up.weight"].T
                half = gu.shape[0] // 2
                y[t] = weight[t] * ((torch.nn.functional.silu(gu[:half]) * gu[half:]) @ w[p + f"moe.experts.{j}.down.weight"].T)
            x = x + y
    return plain_llama.rms_norm(x, w["model.norm.weight"], cfg.eps) @ w["lm_head.weight"].T


def test_toy_architecture_with_routing_another_position_encoding_and_another_norm(tmp_path):
    """32-bit only: the toy router takes the larger of two softmax values, and a 16-bit rounding of its input
    can turn a near tie; the point here is that the parts are registered, built, cached and stepped."""
    from llmserve_triton_kernels_b200 import LLM, SamplingParams
    from llmserve_triton_kernels_b200.config import unregister_architecture
    from llmserve_triton_kernels_b200.engine.batch import StepEntry
    from llmserve_triton_kernels_b200.weights import write_random_model

    register_routed_toy()
    try:
        cfg = RoutedConfig(vocab_size=160, hidden_size=48, intermediate_size=40, num_heads=3, num_kv_heads=1, num_experts=3,
                           slope=1.5, eps=1e-5, max_positions=80)
        folder = write_random_model(tmp_path, cfg, seed=5, std=0.08, dtype=torch.float32)
        _, w = plain_llama.read_model(folder)
        assert "model.layers.1.moe.experts.2.down.weight" in w and "model.layers.1.ff_norm.weight" in w
        llm = LLM(folder, dtype="float32", device=DEV, block_size=4, num_blocks=48, max_batch_size=2, max_num_batched_tokens=32, chunk_size=8)
        a, b = tiny_configs.seeded_tokens(160, [37, 20], 77)
        ref_a, ref_b = routed_plain_forward(cfg, w, a), routed_plain_forward(cfg, w, b)
        step = llm.step_function
        got_a, got_b = [], []
        ia = ib = 0
        for na, nb in ((9, 1), (2, 7), (13, 2), (1, 1), (12, 9)):
            entries = []
            ta, tb = a[ia : ia + na], b[ib : ib + nb]
            if ta:
                entries.append(StepEntry("a", ta, list(range(len(ta)))))
            if tb:
                entries.append(StepEntry("b", tb, list(range(len(tb)))))
            out = step(entries).float().cpu()
            got_a.append(out[: len(ta)])
            got_b.append(out[len(ta) :])
            ia, ib = ia + na, ib + nb
        for got, ref in ((torch.cat(got_a), ref_a), (torch.cat(got_b), ref_b)):
            assert got.shape == ref.shape
            assert float((got - ref).abs().max()) <= 5e-5 * float(ref.abs().max())
        llm.cache.free_request("a")
        llm.cache.free_request("b")
        llm.cache.check()
        out = llm.generate([a[:11]], SamplingParams(max_new_tokens=5))[0]
        tokens = list(a[:11])
        for _ in range(5):
            tokens.append(int(torch.argmax(routed_plain_forward(cfg, w, tokens)[-1])))
        assert out.token_ids == tokens[11:]
    finally:
        unregister_architecture("RoutedToyForCausalLM")


@pytest.mark.parametrize("dtype,storage,rtol", [("float32", torch.float32, 3e-5), ("bfloat16", torch.bfloat16, 3e-2)])
def test_llama_parts_in_another_order_windows_repeats_and_shared_caches(dtype, storage, rtol, model_folder):
    """The Llama parts under an order that Llama does not have, against plain_llama.forward with the
    same windows and order."""
    from llmserve_triton_kernels_b200.cache import CacheManager
    from llmserve_triton_kernels_b200.config import LlamaConfig
    from llmserve_triton_kernels_b200.engine.batch import StepEntry
    from llmserve_triton_kernels_b200.engine.step import StepFunction
    from llmserve_triton_kernels_b200.models.llama import llama_plan
    from llmserve_triton_kernels_b200.models.model import Model
    from llmserve_triton_kernels_b200.models.plan import LayerRun, LayerSpec, ModelPlan
    from llmserve_triton_kernels_b200.parts import PartSpec
    from llmserve_triton_kernels_b200.weights import check_tensors, read_safetensors
    from dataclasses import replace

    cfg_dict, seed, _, _ = tiny_configs.TINY["b"]
    folder = model_folder(cfg_dict, seed, storage)
    plain_cfg, w = plain_llama.read_model(folder)
    base = llama_plan(LlamaConfig.from_dict(cfg_dict))
    windows = [None, 9, None]
    layers = []
    for spec, window in zip(base.layers, windows):
        mixer = PartSpec(spec.mixer.kind, {**spec.mixer.params, "window": window}, spec.mixer.prefix)
        layers.append(spec.replace(mixer=mixer))
    schedule = (LayerRun(0), LayerRun(1), LayerRun(1), LayerRun(2), LayerRun(0))  # layer 1 twice, layer 0 again at the end
    plan = replace(base, layers=tuple(layers), schedule=schedule)
    model = Model(plan, torch.float32 if dtype == "float32" else torch.bfloat16, DEV)
    tensors = read_safetensors(folder)
    check_tensors(tensors, model.tensor_specs(), model.ignored_tensor_names())
    model.bind(tensors)
    cache = CacheManager(model.cache_specs(), plan.schedule, page_size=8, num_pages=24, max_requests=2, dtype=model.dtype, device=DEV)
    assert sorted(len(g.entries) for g in cache.groups) == [2, 3]  # two windowed runs of layer 1; three full caches
    step = StepFunction(model, cache)
    tokens = tiny_configs.seeded_tokens(cfg_dict["vocab_size"], [50], 61)[0]
    ref = plain_llama.forward(plain_cfg, w, tokens, windows=windows, schedule=[(r.layer, r.cache_of) for r in schedule])
    got, i = [], 0
    for n in (13, 2, 1, 16, 1, 1, 9, 7):
        got.append(step([StepEntry("q", tokens[i : i + n], list(range(n)))]).float().cpu().clone())
        i += n
    got = torch.cat(got)
    assert float((got - ref).abs().max()) <= rtol * float(ref.abs().max())
