"""Safetensors reading and writing, weight errors, random weights (no GPU)."""
import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file as st_save

from rust_mlx_b200.config import Qwen3Config
from rust_mlx_b200.registry import build_model_spec
from rust_mlx_b200.weights import SafetensorsFile, WeightsError, load_tensors, save_file, write_random_model
from rust_mlx_b200.weights.random_init import draw
import tiny


def test_own_writer_is_read_by_the_safetensors_package_and_back(tmp_path):
    t = {"a.weight": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "table": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    p = str(tmp_path / "x.safetensors")
    save_file(t, p)
    theirs = load_file(p)
    for k in t:
        assert theirs[k].dtype == t[k].dtype and torch.equal(theirs[k], t[k])
    p2 = str(tmp_path / "y.safetensors")
    st_save(t, p2)
    f = SafetensorsFile(p2)
    for k in t:
        got = f.tensor(k)
        assert got.dtype == t[k].dtype and torch.equal(got, t[k])


def test_random_model_folder_is_reproducible_and_keyed_by_name(tmp_path):
    cfg = Qwen3Config.from_dict(tiny.TINY_B)
    a = write_random_model(cfg, str(tmp_path / "a"), seed=5, store_dtype="float32")
    b = write_random_model(cfg, str(tmp_path / "b"), seed=5, store_dtype="float32")
    c = write_random_model(cfg, str(tmp_path / "c"), seed=6, store_dtype="float32")
    ta, tb, tc = (load_file(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    assert set(ta) == {s.name for s in build_model_spec(cfg).all_param_specs()}
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert not torch.equal(ta["lm_head.weight"], tc["lm_head.weight"])
    # the recipe: matrices N(0, 0.02), norm weights 1 + N(0, 0.05)
    assert abs(ta["model.embed_tokens.weight"].std().item() - 0.02) < 2e-3
    norm = ta["model.layers.1.input_layernorm.weight"]
    assert abs(norm.mean().item() - 1.0) < 0.03 and 0.02 < norm.std().item() < 0.08
    # a tensor's values depend on (seed, name) only
    spec = [s for s in build_model_spec(cfg).all_param_specs() if s.name == "model.norm.weight"][0]
    assert torch.equal(draw(spec, 5), ta["model.norm.weight"])
    assert json.load(open(os.path.join(a, "config.json")))["vocab_size"] == 509
    bf = write_random_model(cfg, str(tmp_path / "bf"), seed=5, store_dtype="bfloat16")
    tbf = load_file(os.path.join(bf, "model.safetensors"))
    assert tbf["lm_head.weight"].dtype == torch.bfloat16
    assert tbf["model.norm.weight"].dtype == torch.float32   # stored in 32-bit, stays so
    assert torch.equal(tbf["lm_head.weight"], ta["lm_head.weight"].to(torch.bfloat16))


def test_random_numbers_are_a_function_of_key_and_index():
    """The generator against its definition restated with Python integers: element i takes outputs 3i+1..3i+3 of
    SplitMix64 keyed by ``key``, adds their twelve 16-bit pieces, centres and scales once in float32.  Numbers made
    in one piece and in pieces (the generator works in chunks) are the same."""
    import numpy as np
    from rust_mlx_b200.weights import random_init
    mask = (1 << 64) - 1

    def mix(z):
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        return z ^ (z >> 31)
    key = 0xFEDCBA9876543210
    scale = np.float32(0.02 / (2.0 * (65536.0 ** 2 - 1.0) ** 0.5))
    x = random_init.normal(key, 5000, 0.02)
    for i in (0, 1, 2, 77, 4999):
        total = 0
        for k in (1, 2, 3):
            h = mix((key + (3 * i + k) * 0x9E3779B97F4A7C15) & mask)
            total += sum((h >> s) & 0xFFFF for s in (0, 16, 32, 48))
        assert np.float32(x[i].item()) == np.float32(2 * total - 12 * 65535) * scale, i
    old = random_init._CHUNK
    random_init._CHUNK = 1024
    try:
        assert torch.equal(random_init.normal(key, 5000, 0.02), x)
    finally:
        random_init._CHUNK = old
    big = random_init.normal(3, 200000, 1.0)
    assert abs(big.mean().item()) < 0.01 and abs(big.std().item() - 1.0) < 0.01
    assert abs((big ** 4).mean().item() - 2.9) < 0.1           # a sum of twelve uniform numbers: kurtosis 2.9


@pytest.mark.gpu
def test_random_weights_are_the_same_on_the_gpu_as_in_a_folder(tmp_path):
    """``Engine(config, random_weights=True)`` draws on the GPU what ``write_random_model`` draws on the CPU for the
    same seed: bit for bit, in both held dtypes, and so the command line's ``--random-weights`` generates what the
    written folder generates."""
    import subprocess
    import sys
    from rust_mlx_b200.weights import random_tensors
    cfg = Qwen3Config.from_dict(tiny.TINY_D)
    specs = build_model_spec(cfg).all_param_specs()
    for store, held in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
        folder = write_random_model(cfg, str(tmp_path / store), seed=9, store_dtype=store)
        disk = load_tensors(folder, specs, held, "cuda:0")
        made = random_tensors(specs, 9, held, "cuda:0")
        assert set(disk) == set(made)
        for k in disk:
            assert disk[k].dtype == made[k].dtype and torch.equal(disk[k], made[k]), k
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ids = str(tmp_path / "p.json")
    json.dump([5, 9, 300, 41, 7], open(ids, "w"))
    outs = []
    for extra in ([], ["--random-weights"]):
        out = str(tmp_path / f"r{len(extra)}.json")
        subprocess.run([sys.executable, os.path.join(root, "bin", "infer"), "--model", folder, "--prompt-ids", ids,
                        "--max-tokens", "8", "--runs", "1", "--warmup-tokens", "1", "--ignore-eos", "--seed", "9",
                        "--output", out] + extra, check=True, timeout=600)
        outs.append(json.load(open(out))["runs"][0]["tokens"])
    assert outs[0] == outs[1] and len(outs[0]) == 8


def test_dtypes_held(tmp_path):
    cfg = Qwen3Config.from_dict(tiny.TINY_A)
    folder = write_random_model(cfg, str(tmp_path / "m"), seed=1, store_dtype="bfloat16")
    specs = build_model_spec(cfg).all_param_specs()
    t16 = load_tensors(folder, specs, torch.bfloat16, "cpu")
    t32 = load_tensors(folder, specs, torch.float32, "cpu")
    assert t16["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert t16["model.layers.0.input_layernorm.weight"].dtype == torch.float32
    assert t32["model.layers.0.mlp.up_proj.weight"].dtype == torch.float32
    assert torch.equal(t32["model.layers.0.mlp.up_proj.weight"], t16["model.layers.0.mlp.up_proj.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = Qwen3Config.from_dict(tiny.TINY_B)
    folder = write_random_model(cfg, str(tmp_path / "m"), seed=1, store_dtype="float32")
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    del t["model.layers.2.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(4)
    t["model.layers.1.self_attn.k_proj.weight"] = torch.zeros(5, 96)
    t["lm_head.weight"] = torch.zeros(509, 96, dtype=torch.int32)
    st_save(t, path)
    specs = build_model_spec(cfg).all_param_specs()
    with pytest.raises(WeightsError) as e:
        load_tensors(folder, specs, torch.float32, "cpu")
    err = e.value
    assert err.missing == ["model.layers.2.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary.inv_freq"]
    assert len(err.wrong) == 2
    msg = str(err)
    for word in ("missing", "unexpected", "model.layers.1.self_attn.k_proj.weight has shape [5, 96]",
                 "needs [64, 96]", "lm_head.weight is stored as torch.int32"):
        assert word in msg


def test_duplicates_across_shards_and_index_file(tmp_path):
    cfg = Qwen3Config.from_dict(tiny.TINY_A)
    folder = write_random_model(cfg, str(tmp_path / "m"), seed=1, store_dtype="float32")
    t = load_file(os.path.join(folder, "model.safetensors"))
    specs = build_model_spec(cfg).all_param_specs()
    st_save({"model.norm.weight": t["model.norm.weight"]}, os.path.join(folder, "extra.safetensors"))
    with pytest.raises(WeightsError) as e:
        load_tensors(folder, specs, torch.float32, "cpu")
    assert e.value.duplicate == ["model.norm.weight"]
    # with an index only the shards it names are read (src/weights.rs:25-33)
    json.dump({"weight_map": {k: "model.safetensors" for k in t}}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    got = load_tensors(folder, specs, torch.float32, "cpu")
    assert torch.equal(got["model.norm.weight"], t["model.norm.weight"])


def test_a_tied_checkpoint_may_carry_its_head(tmp_path):
    cfg = Qwen3Config.from_dict(tiny.TINY_A)
    folder = write_random_model(cfg, str(tmp_path / "m"), seed=1, store_dtype="float32")
    path = os.path.join(folder, "model.safetensors")
    t = load_file(path)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    st_save(t, path)
    spec = build_model_spec(cfg)
    load_tensors(folder, spec.all_param_specs(), torch.float32, "cpu", spec.ignored_tensors)


def test_folder_without_weights(tmp_path):
    cfg = Qwen3Config.from_dict(tiny.TINY_A)
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_A))
    with pytest.raises(WeightsError) as e:
        load_tensors(str(tmp_path), build_model_spec(cfg).all_param_specs(), torch.float32, "cpu")
    assert "no safetensors" in str(e.value)
