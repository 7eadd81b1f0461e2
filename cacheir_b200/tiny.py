"""Tiny random Llama-shaped model on disk (config.json + weights.npz).

Same recipe as the reference's `create_tiny_model`
(cacheir/importers/tiny.py:9-65): one `np.random.default_rng(seed)` stream,
every matrix `standard_normal(shape) * 0.02` as float32, drawn in the order
embed, lm_head, then per layer q, k, v, o, gate, up, down; norm weights are
ones. Used for the reference's CPU-runnable configuration and by the tests.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np


def tiny_model_tensors(*, seed: int = 7, vocab_size: int = 64, hidden_size: int = 32, intermediate_size: int = 64,
                       num_layers: int = 2, num_attention_heads: int = 4, num_key_value_heads: int = 2
                       ) -> dict[str, np.ndarray]:
    rng = np.random.default_rng(seed)

    def normal(shape: tuple[int, ...]) -> np.ndarray:
        return (rng.standard_normal(shape) * 0.02).astype(np.float32)

    weights: dict[str, np.ndarray] = {
        "model.embed_tokens.weight": normal((vocab_size, hidden_size)),
        "model.norm.weight": np.ones((hidden_size,), dtype=np.float32),
        "lm_head.weight": normal((vocab_size, hidden_size)),
    }
    head_dim = hidden_size // num_attention_heads
    kv_dim = num_key_value_heads * head_dim
    for layer in range(num_layers):
        p = f"model.layers.{layer}"
        weights[f"{p}.input_layernorm.weight"] = np.ones((hidden_size,), dtype=np.float32)
        weights[f"{p}.self_attn.q_proj.weight"] = normal((hidden_size, hidden_size))
        weights[f"{p}.self_attn.k_proj.weight"] = normal((kv_dim, hidden_size))
        weights[f"{p}.self_attn.v_proj.weight"] = normal((kv_dim, hidden_size))
        weights[f"{p}.self_attn.o_proj.weight"] = normal((hidden_size, hidden_size))
        weights[f"{p}.post_attention_layernorm.weight"] = np.ones((hidden_size,), dtype=np.float32)
        weights[f"{p}.mlp.gate_proj.weight"] = normal((intermediate_size, hidden_size))
        weights[f"{p}.mlp.up_proj.weight"] = normal((intermediate_size, hidden_size))
        weights[f"{p}.mlp.down_proj.weight"] = normal((hidden_size, intermediate_size))
    return weights


def tiny_model_config(*, vocab_size: int = 64, hidden_size: int = 32, intermediate_size: int = 64, num_layers: int = 2,
                      num_attention_heads: int = 4, num_key_value_heads: int = 2) -> dict[str, object]:
    return {
        "architectures": ["CacheIRTinyForCausalLM"],
        "hidden_size": hidden_size,
        "intermediate_size": intermediate_size,
        "num_hidden_layers": num_layers,
        "num_attention_heads": num_attention_heads,
        "num_key_value_heads": num_key_value_heads,
        "vocab_size": vocab_size,
        "max_position_embeddings": 256,
        "rope_theta": 10000.0,
        "rms_norm_eps": 1e-5,
        "torch_dtype": "float32",
        "tie_word_embeddings": False,
    }


def create_tiny_model(path: str | Path, *, seed: int = 7, **shape) -> Path:
    out = Path(path)
    out.mkdir(parents=True, exist_ok=True)
    (out / "config.json").write_text(json.dumps(tiny_model_config(**shape), indent=2), encoding="utf-8")
    np.savez(out / "weights.npz", **tiny_model_tensors(seed=seed, **shape))
    vocab = shape.get("vocab_size", 64)
    (out / "tokenizer_config.json").write_text(json.dumps({"type": "byte_mod", "vocab_size": vocab}, indent=2), encoding="utf-8")
    return out
