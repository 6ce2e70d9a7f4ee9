"""The Qwen3 dense decoder put together from parts (src/dense.rs:306-398).

Tensor names are the checkpoint's (src/dense.rs:335-367).  Every layer is a
pre-norm block of grouped-query attention with per-head q/k RMSNorm and rotary
positions, and a SwiGLU feed-forward; a layer whose kind is "sliding_attention"
gets a window.  The head is tied to the embedding when the configuration says so.
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..parts.attention import AttentionMixer
from ..parts.block import PreNormBlock
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.feedforward import SwiGLUFeedForward
from ..parts.norm import RMSNorm
from ..parts.position import RotaryEmbedding
from ..registry import register_architecture
from .spec import ModelSpec, default_schedule


def build_qwen3(config: Qwen3Config) -> ModelSpec:
    c = config
    rope = RotaryEmbedding(c.head_dim, c.rope_theta, scaling=c.rope_scaling_parameters())
    embedding = TokenEmbedding("model.embed_tokens.weight", c.vocab_size, c.hidden_size)
    blocks = []
    for i, kind in enumerate(c.attention_kinds()):
        p = f"model.layers.{i}"
        mixer = AttentionMixer(f"{p}.self_attn", c.hidden_size, c.num_attention_heads, c.num_key_value_heads,
                               c.head_dim, rope, qk_norm_eps=c.rms_norm_eps,
                               window=c.sliding_window if kind == "sliding_attention" else 0, bias=c.attention_bias)
        blocks.append(PreNormBlock(RMSNorm(f"{p}.input_layernorm.weight", c.hidden_size, c.rms_norm_eps), mixer,
                                   RMSNorm(f"{p}.post_attention_layernorm.weight", c.hidden_size, c.rms_norm_eps),
                                   SwiGLUFeedForward(f"{p}.mlp", c.hidden_size, c.intermediate_size)))
    if c.tie_word_embeddings:
        head = OutputHead(c.vocab_size, c.hidden_size, tied_to=embedding)
    else:
        head = OutputHead(c.vocab_size, c.hidden_size, name="lm_head.weight")
    spec = ModelSpec(config=c, embedding=embedding, blocks=blocks, schedule=default_schedule(len(blocks)),
                     final_norm=RMSNorm("model.norm.weight", c.hidden_size, c.rms_norm_eps), head=head,
                     ignored_tensors=("lm_head.weight",) if c.tie_word_embeddings else (),
                     vocab_size=c.vocab_size, eos_token_ids=tuple(c.eos_token_id))
    spec.check_schedule()
    return spec


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3, model_types=("qwen3",))
