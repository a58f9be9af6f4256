"""Named config.json dictionaries for the random-weights mode.  They are data handed to the
configuration class like any model folder's config.json; nothing in the engine reads them.

``tiny`` has the sizes of the reference's ``ModelConfig.tiny()`` (src/llmserve/config.py:26-37);
``tinyllama-1.1b`` those of its defaults (src/llmserve/config.py:10-20).
"""

from __future__ import annotations


def _llama(**kw) -> dict:
    base = {
        "architectures": ["LlamaForCausalLM"],
        "model_type": "llama",
        "hidden_act": "silu",
        "rope_theta": 10000.0,
        "rms_norm_eps": 1e-5,
        "tie_word_embeddings": False,
    }
    base.update(kw)
    return base


PRESETS: dict[str, dict] = {
    "tiny": _llama(
        vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, max_position_embeddings=512,
    ),
    "tinyllama-1.1b": _llama(
        vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22, num_attention_heads=32,
        num_key_value_heads=4, max_position_embeddings=2048,
    ),
    "llama2-7b": _llama(
        vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
        num_key_value_heads=32, max_position_embeddings=4096,
    ),
    "llama3-8b": _llama(
        vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
        num_key_value_heads=8, max_position_embeddings=8192, rope_theta=500000.0,
    ),
}
