"""Named configurations for the random-weights mode: each is the content of a config.json, as
data.  Nothing in the library reads a size from here; a preset only saves writing the file.

The three full sizes are the published layer sizes of Mistral 7B v0.1 and v0.3 and of Mistral
NeMo 12B; the two tiny ones differ from each other in every size and option (heads and groups,
head size against hidden size, window, rope base, norm epsilon) and run anywhere in seconds.
The reference has one built-in default, the path of its Mistral 7B file (src/main.rs:26-32).
"""
from __future__ import annotations

from typing import Dict

_MISTRAL = {"architectures": ["MistralForCausalLM"], "model_type": "mistral", "hidden_act": "silu",
            "tie_word_embeddings": False, "bos_token_id": 1, "eos_token_id": 2}

PRESETS: Dict[str, dict] = {
    "7b-v0.1": dict(_MISTRAL, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                    num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=32000,
                    rope_theta=10000.0, sliding_window=4096, rms_norm_eps=1e-5, max_position_embeddings=32768),
    "7b-v0.3": dict(_MISTRAL, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
                    num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=32768,
                    rope_theta=1000000.0, sliding_window=None, rms_norm_eps=1e-5, max_position_embeddings=32768),
    "nemo-12b": dict(_MISTRAL, num_hidden_layers=40, hidden_size=5120, num_attention_heads=32,
                     num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=131072,
                     rope_theta=1000000.0, sliding_window=None, rms_norm_eps=1e-5, max_position_embeddings=131072),
    "tiny-a": dict(_MISTRAL, num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=16, intermediate_size=192, vocab_size=256,
                   rope_theta=10000.0, sliding_window=16, rms_norm_eps=1e-5, max_position_embeddings=512),
    "tiny-b": dict(_MISTRAL, num_hidden_layers=3, hidden_size=96, num_attention_heads=6,
                   num_key_value_heads=1, head_dim=32, intermediate_size=160, vocab_size=384,
                   rope_theta=1000000.0, sliding_window=None, rms_norm_eps=1e-6, max_position_embeddings=1024),
}


def preset(name: str) -> dict:
    """A copy of the named configuration (a config.json-style dict)."""
    try:
        return dict(PRESETS[name])
    except KeyError:
        raise KeyError(f"unknown preset {name!r}; presets: {sorted(PRESETS)}") from None
