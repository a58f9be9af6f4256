"""The small configurations the tests run: two Llama models that differ in every size and
option, as plain config.json dictionaries, and their seeded prompts."""

from __future__ import annotations

import torch

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 256,
    "hidden_size": 64,
    "intermediate_size": 172,
    "num_hidden_layers": 2,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "max_position_embeddings": 128,
    "rope_theta": 10000.0,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
}
TINY_A_SEED, TINY_A_PROMPT_SEED, TINY_A_PROMPT_LENS = 0, 1, (5, 11, 17)

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "vocab_size": 384,
    "hidden_size": 96,
    "intermediate_size": 256,
    "num_hidden_layers": 3,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "max_position_embeddings": 256,
    "rope_theta": 500000.0,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True,
    "hidden_act": "silu",
}
TINY_B_SEED, TINY_B_PROMPT_SEED, TINY_B_PROMPT_LENS = 2, 3, (1, 7, 23, 40)

# Head sizes 64 and 128: the sizes the one-kernel decode step takes (the two above go kernel by kernel)
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 320, "hidden_size": 128, "intermediate_size": 200,
    "num_hidden_layers": 2, "num_attention_heads": 2, "num_key_value_heads": 1, "max_position_embeddings": 192,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "hidden_act": "silu",
}
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 288, "hidden_size": 384, "intermediate_size": 264,
    "num_hidden_layers": 3, "num_attention_heads": 3, "num_key_value_heads": 3, "max_position_embeddings": 160,
    "rope_theta": 50000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "hidden_act": "silu",
}

TINY = {
    "a": (TINY_A, TINY_A_SEED, TINY_A_PROMPT_SEED, TINY_A_PROMPT_LENS),
    "b": (TINY_B, TINY_B_SEED, TINY_B_PROMPT_SEED, TINY_B_PROMPT_LENS),
    "c": (TINY_C, 4, 5, (3, 9, 21)),
    "d": (TINY_D, 6, 7, (2, 14, 30)),
}


def seeded_tokens(vocab: int, lengths, seed: int) -> list[list[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


def prompts(name: str) -> list[list[int]]:
    cfg, _, prompt_seed, lens = TINY[name]
    return seeded_tokens(cfg["vocab_size"], lens, prompt_seed)
