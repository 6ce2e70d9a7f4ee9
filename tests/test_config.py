"""Configuration and registry (no GPU)."""
import json
import math
import os

import pytest
import torch

from rust_mlx_b200.config import ConfigError, Qwen3Config
from rust_mlx_b200.registry import (find_architecture, known_architectures, load_config, register_architecture,
                                    unregister_architecture, build_model_spec)
import tiny


def test_reads_every_key_of_both_tiny_configs():
    a = Qwen3Config.from_dict(tiny.TINY_A)
    b = Qwen3Config.from_dict(tiny.TINY_BW)
    assert Qwen3Config.from_dict(tiny.TINY_B).attention_kinds() == ("full_attention",) * 3
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (2, 64, 4, 2, 16)
    assert (b.intermediate_size, b.vocab_size, b.rope_theta, b.rms_norm_eps) == (160, 509, 1e6, 1e-5)
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert a.attention_kinds() == ("full_attention",) * 2
    assert b.attention_kinds() == ("full_attention", "sliding_attention", "sliding_attention")


def test_defaults_follow_the_reference():
    raw = {k: v for k, v in tiny.TINY_A.items() if k not in ("rope_theta", "head_dim", "tie_word_embeddings")}
    c = Qwen3Config.from_dict(raw)
    assert c.rope_theta == 1e6            # src/dense.rs:323-332
    assert c.head_dim == 64 // 4
    assert c.tie_word_embeddings is False
    c = Qwen3Config.from_dict(dict(raw, rope_parameters={"rope_theta": 5000.0}))
    assert c.rope_theta == 5000.0
    c = Qwen3Config.from_dict(dict(raw, eos_token_id=7))
    assert c.eos_token_id == (7,)
    c = Qwen3Config.from_dict(dict(raw, eos_token_id=[7, 9]))
    assert c.eos_token_id == (7, 9)


def test_all_problems_are_reported_at_once():
    raw = dict(tiny.TINY_A)
    del raw["hidden_size"]
    raw["vocab_size"] = "many"
    raw["rms_norm_eps"] = None
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(raw)
    msg = str(e.value)
    assert "hidden_size" in msg and "vocab_size" in msg and "rms_norm_eps" in msg


@pytest.mark.parametrize("change, word", [
    (dict(num_key_value_heads=3), "multiple"),
    (dict(head_dim=15), "even"),
    (dict(model_type="llama"), "model_type"),
    (dict(rope_scaling={"rope_type": "llama3", "factor": 4}), "rope_scaling"),
    (dict(rope_scaling={"rope_type": "yarn"}), "factor"),
    (dict(rope_scaling={"type": "linear", "factor": 0.5}), "factor"),
    (dict(rope_scaling={"rope_type": "yarn", "factor": 2}, max_position_embeddings=0), "original_max_position_embeddings"),
    (dict(use_sliding_window=True, sliding_window=0), "sliding_window"),
    (dict(use_sliding_window=True, sliding_window=8, layer_types=["full_attention"]), "layer_types"),
    (dict(num_hidden_layers=0), "positive"),
])
def test_invalid_configurations_are_refused(change, word):
    with pytest.raises(ConfigError) as e:
        Qwen3Config.from_dict(dict(tiny.TINY_A, **change))
    assert word in str(e.value)


def test_registry_picks_by_architecture_then_model_type(tmp_path):
    assert "Qwen3ForCausalLM" in known_architectures()
    assert find_architecture({"architectures": ["Qwen3ForCausalLM"]}).config_class is Qwen3Config
    assert find_architecture({"model_type": "qwen3"}).config_class is Qwen3Config
    with pytest.raises(ConfigError) as e:
        find_architecture({"architectures": ["NoSuchModel"], "model_type": "qwen3"})
    assert "NoSuchModel" in str(e.value) and "Qwen3ForCausalLM" in str(e.value)
    p = tmp_path / "config.json"
    p.write_text(json.dumps(tiny.TINY_B))
    cfg = load_config(str(tmp_path))
    assert isinstance(cfg, Qwen3Config) and cfg.vocab_size == 509
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "nowhere"))


def test_round_trip_through_to_dict():
    for raw in (tiny.TINY_A, tiny.TINY_B):
        c = Qwen3Config.from_dict(raw)
        again = Qwen3Config.from_dict(json.loads(json.dumps(c.to_dict())))
        assert again == c


def test_model_spec_takes_sizes_from_configuration_only():
    for raw in (tiny.TINY_A, tiny.TINY_B):
        c = Qwen3Config.from_dict(raw)
        spec = build_model_spec(c)
        shapes = {s.name: s.shape for s in spec.all_param_specs()}
        hd, nq, nkv = c.head_dim, c.num_attention_heads, c.num_key_value_heads
        assert shapes["model.embed_tokens.weight"] == (c.vocab_size, c.hidden_size)
        assert shapes["model.layers.0.self_attn.q_proj.weight"] == (nq * hd, c.hidden_size)
        assert shapes["model.layers.0.self_attn.k_proj.weight"] == (nkv * hd, c.hidden_size)
        assert shapes["model.layers.0.self_attn.o_proj.weight"] == (c.hidden_size, nq * hd)
        assert shapes["model.layers.0.self_attn.q_norm.weight"] == (hd,)
        assert shapes["model.layers.0.mlp.down_proj.weight"] == (c.hidden_size, c.intermediate_size)
        assert ("lm_head.weight" in shapes) == (not c.tie_word_embeddings)
        assert len(spec.blocks) == c.num_hidden_layers == len(spec.schedule)
        windows = [b.mixer.window for b in spec.blocks]
        assert windows == [c.sliding_window if k == "sliding_attention" else 0 for k in c.attention_kinds()]


def test_an_architecture_can_be_added_and_removed():
    register_architecture("ToyForCausalLM", Qwen3Config, lambda cfg: "built", model_types=("toy",))
    try:
        assert find_architecture({"architectures": ["ToyForCausalLM"]}).build(None) == "built"
    finally:
        unregister_architecture("ToyForCausalLM")
    assert "ToyForCausalLM" not in known_architectures()


def test_projection_bias_and_scaled_rotation_are_read():
    from rust_mlx_b200.registry import build_model_spec
    cfg = Qwen3Config.from_dict(dict(tiny.TINY_A, attention_bias=True,
                                     rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32}))
    spec = build_model_spec(cfg)
    names = {s.name: s for s in spec.all_param_specs()}
    assert names["model.layers.1.self_attn.k_proj.bias"].shape == (2 * 16,)
    assert names["model.layers.0.self_attn.o_proj.bias"].optional and not names["model.layers.0.self_attn.q_proj.bias"].optional
    mixer = spec.blocks[0].mixer
    plain_table = 10000.0 ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16)
    assert torch.equal(mixer.position._table[:1], plain_table[:1].float())           # the fastest pair keeps its frequency
    assert torch.allclose(mixer.position._table[-1:], (plain_table[-1:] / 4).float())   # the slowest is divided by the factor
    assert abs(mixer.scale - 16 ** -0.5 * (0.1 * math.log(4.0) + 1.0) ** 2) < 1e-12
    # newer checkpoints keep theta and the scaling together
    cfg2 = Qwen3Config.from_dict({k: v for k, v in dict(tiny.TINY_A, rope_parameters={
        "rope_theta": 5e4, "rope_type": "linear", "factor": 2.0}).items() if k != "rope_theta"})
    assert cfg2.rope_theta == 5e4 and cfg2.rope_scaling_parameters()["factor"] == 2.0
    linear = build_model_spec(cfg2).blocks[0].mixer.position
    assert torch.allclose(linear._table.double(), 5e4 ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16) / 2, rtol=1e-6)
    assert linear.score_scale == 1.0
