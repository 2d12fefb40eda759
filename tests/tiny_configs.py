"""Small configurations of the architecture for the tests. They differ in every size and
option: layers, width, head counts and groups, head size, feed-forward width, vocabulary,
rope base, eps, tied or untied head, bias, window, unrotated layers, page size."""
import os

import torch

TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    intermediate_size=128, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=True, attention_bias=False, max_position_embeddings=512, hidden_act="silu",
    eos_token_id=255)
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=8, num_key_value_heads=2, head_dim=32,
    intermediate_size=224, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
    tie_word_embeddings=False, attention_bias=False, max_position_embeddings=1024, hidden_act="silu",
    eos_token_id=[382, 383])
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=4, hidden_size=80, num_attention_heads=6, num_key_value_heads=3, head_dim=48,
    intermediate_size=176, vocab_size=333, rope_theta=500000.0, rms_norm_eps=3e-6,
    tie_word_embeddings=False, attention_bias=True, max_position_embeddings=640, hidden_act="silu",
    use_sliding_window=True, sliding_window=24, max_window_layers=2, no_rope_layers=[False, False, False, True],
    eos_token_id=1)

# Heads of 128 elements, a feed-forward width that is a multiple of 128 and a width that is a multiple
# of 8: the sizes at which the bfloat16 engine takes its tcgen05 kernels (attention over long portions,
# products with fused epilogues) and the vectorised rotation kernel.
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
    intermediate_size=640, vocab_size=520, rope_theta=1000000.0, rms_norm_eps=1e-6,
    tie_word_embeddings=False, attention_bias=False, max_position_embeddings=2048, hidden_act="silu",
    eos_token_id=519)

# Heads wider than 128 elements and no power of two (the bfloat16 engine then takes its generic attention
# kernels), one key head for three query heads, pages of 4 keys, a width and a vocabulary that are odd multiples.
TINY_F = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=72, num_attention_heads=3, num_key_value_heads=1, head_dim=160,
    intermediate_size=200, vocab_size=291, rope_theta=20000.0, rms_norm_eps=2e-6,
    tie_word_embeddings=True, attention_bias=False, max_position_embeddings=700, hidden_act="silu",
    eos_token_id=[7])

# Sizes that are multiples of nothing useful: a width of 70, a feed-forward width of 150, a prime vocabulary, five
# heads that each have their own key head (no grouping): no vectorised or tensor-core fast path applies as it stands.
TINY_G = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3",
    num_hidden_layers=2, hidden_size=70, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
    intermediate_size=150, vocab_size=257, rope_theta=10000.0, rms_norm_eps=1e-5,
    tie_word_embeddings=False, attention_bias=True, max_position_embeddings=300, hidden_act="silu",
    eos_token_id=3)

# name -> (config.json, seed, sigma of matrices, page size); E is D with pages of 64 keys
TINY = {"A": (TINY_A, 0, 0.02, 16), "B": (TINY_B, 1, 0.03, 8), "C": (TINY_C, 5, 0.05, 16),
        "D": (TINY_D, 6, 0.04, 16), "E": (TINY_D, 6, 0.04, 64), "F": (TINY_F, 9, 0.05, 4),
        "G": (TINY_G, 10, 0.05, 16)}


def write_tiny_model(name: str, folder: str, sigma_scale: float = 1.0, norm_dtype=None) -> str:
    """Write the tiny model ``name`` into ``folder`` with the package's random-weights mode."""
    from llm_rs_b200.config import Qwen3Config
    from llm_rs_b200.weights import write_random_model
    raw, seed, sigma, _ = TINY[name]
    cfg = Qwen3Config.from_dict(raw)
    return write_random_model(os.path.join(folder, f"tiny_{name}"), cfg, seed=seed, sigma=sigma * sigma_scale,
                              norm_jitter=0.1, dtype=torch.bfloat16, norm_dtype=norm_dtype)
