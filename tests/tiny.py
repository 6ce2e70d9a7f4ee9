"""Tiny configurations and helpers shared by the tests.

A and B differ in every size and option: layers, width, head counts and group size,
head_dim (A: heads * head_dim equals the width, B: it does not), feed-forward width,
vocabulary (B: odd), rope_theta, eps, tied or untied head, page size.  "Bw" is B with a
sliding window in its upper layers.
"""
import os
import random

import torch

TINY_A = dict(
    model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=64,
    num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096)
PAGE_A = 16

TINY_B = dict(
    model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=96,
    num_attention_heads=6, num_key_value_heads=2, head_dim=32, intermediate_size=160, vocab_size=509,
    rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=4096)
PAGE_B = 8
# B with a window of 20 keys in layers 1 and 2 (layer 0 attends to everything)
TINY_BW = dict(TINY_B, use_sliding_window=True, sliding_window=20, max_window_layers=1)

# C and D have the head sizes of real checkpoints, so that the engine's bfloat16 replay goes through the kernels
# that serve them (TMA-fed attention at 64 and 128, tcgen05 prompt attention at 128, the tcgen05 products):
# C: head 64, group 3, a window; D: head 128, group 4, widths that are multiples of 64 (fused gate/up blocks).
TINY_C = dict(
    model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=136,
    num_attention_heads=6, num_key_value_heads=2, head_dim=64, intermediate_size=200, vocab_size=333,
    rope_theta=50000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096,
    use_sliding_window=True, sliding_window=70, max_window_layers=1)
PAGE_C = 32

TINY_D = dict(
    model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=256,
    num_attention_heads=8, num_key_value_heads=2, head_dim=128, intermediate_size=384, vocab_size=520,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096)
PAGE_D = 64

# E: head 128 with a window and small pages (four copies a key tile, pages handed back while a prompt runs), group 2
TINY_E = dict(
    model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=3, hidden_size=192,
    num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=320, vocab_size=411,
    rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=4096,
    use_sliding_window=True, sliding_window=100, max_window_layers=1)
PAGE_E = 16

# F: projections with a bias and yarn-scaled rotation (original context 32, so that the ramp lies inside these heads);
# G: D's head size 128 (the decoding attention finishes the projection itself) with a bias and linearly scaled rotation
TINY_F = dict(
    model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=80,
    num_attention_heads=5, num_key_value_heads=5, head_dim=32, intermediate_size=96, vocab_size=301,
    rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096,
    attention_bias=True, rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32})
PAGE_F = 16
TINY_G = dict(TINY_D, attention_bias=True, rope_scaling={"type": "linear", "factor": 8.0})

CONFIGS = {"A": (TINY_A, PAGE_A), "B": (TINY_B, PAGE_B), "Bw": (TINY_BW, PAGE_B), "C": (TINY_C, PAGE_C), "D": (TINY_D, PAGE_D),
           "E": (TINY_E, PAGE_E), "F": (TINY_F, PAGE_F), "G": (TINY_G, PAGE_D)}


def make_folder(tmp_path, raw: dict, seed: int = 0, store: str = "float32") -> str:
    """Write a model folder with the engine's random-weights mode."""
    from rust_mlx_b200.config import Qwen3Config
    from rust_mlx_b200.weights import write_random_model
    folder = os.path.join(str(tmp_path), f"model_{abs(hash(str(sorted(raw.items()))))%10**8}_{seed}_{store}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        write_random_model(Qwen3Config.from_dict(raw), folder, seed=seed, store_dtype=store)
    return folder


def prompts(vocab: int, lengths, seed: int = 1) -> list:
    rng = random.Random(seed)
    return [[rng.randrange(vocab) for _ in range(n)] for n in lengths]


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return (a.double() - b.double()).abs().max().item()


def sharpen(folder: str, factor: float = 2.0) -> str:
    """A copy of ``folder`` whose q_norm and k_norm weights are multiplied by ``factor``.

    With N(0, 0.02) weights every score is near zero and attention is an average over all
    keys: a key that is missing, stale or read from the wrong page changes the result by
    about 1/length and hides in the tolerance.  Scaling both norms by 2 scales scores by
    4, so a few keys carry most of the weight and any wrong key shows."""
    from safetensors.torch import load_file, save_file
    import shutil
    out = folder + f"_sharp{factor}"
    if not os.path.exists(os.path.join(out, "model.safetensors")):
        os.makedirs(out, exist_ok=True)
        shutil.copy(os.path.join(folder, "config.json"), os.path.join(out, "config.json"))
        t = load_file(os.path.join(folder, "model.safetensors"))
        for k in t:
            if k.endswith("q_norm.weight") or k.endswith("k_norm.weight"):
                t[k] = t[k] * factor
        save_file(t, os.path.join(out, "model.safetensors"))
    return out
