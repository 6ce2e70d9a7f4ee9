"""The engine at the layer sizes of Qwen3-8B (hidden 4096, 32 query / 8 kv heads of 128, feed-forward
12288, vocabulary 151936), two layers, random weights: the kernels at the sizes they serve.

float32: logits equal the plain implementation's (run here in float64 on the GPU, with the same
weights), and are bit-identical whole, with the last 32 tokens one by one, in portions and mixed.  bfloat16: every way of cutting stays
within the bfloat16 tolerance of the plain implementation's bfloat16 restatement.
"""
import pytest
import torch

import plain_qwen3 as plain
import replay
import tiny

pytestmark = pytest.mark.gpu

SHAPE_8B = dict(
    model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
    rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096)
LENGTHS = [150, 33, 70, 9]


def engine_and_weights(dtype, tokens, **options):
    from rust_mlx_b200.config import Qwen3Config
    from rust_mlx_b200.engine import Engine
    from rust_mlx_b200.registry import build_model_spec
    from rust_mlx_b200.weights.random_init import random_tensors
    cfg = Qwen3Config.from_dict(SHAPE_8B)
    eng = Engine(cfg, dtype=dtype, random_weights=True, seed=5, max_tokens=tokens, page_size=64, max_requests=4, **options)
    # the same tensors again, by name, for the plain implementation (drawn from (seed, name), so they are equal)
    held = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    tensors = random_tensors(build_model_spec(cfg).all_param_specs(), 5, held, "cuda:0")
    return eng, tensors


@pytest.mark.parametrize("dtype, tuned", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
def test_layer_sizes_of_qwen3_8b(dtype, tuned):
    """``tuned``: the engine times its tcgen05 product against the library's on these two layers' weights when it
    starts (as it does at full depth, where a shape's weights hold far more than the threshold lowered here) and
    runs with what it chose: q/k/v and output projections on the tcgen05 kernel with the tuned number of K
    slices, the choice changing with the padded row count.  The same bound holds, and an engine given the first
    one's table makes the same choices and gives the same bits."""
    reqs = {f"r{i}": p for i, p in enumerate(tiny.prompts(SHAPE_8B["vocab_size"], LENGTHS, seed=3))}
    steps_by_way = {w: getattr(replay, w)(reqs) for w in ("whole", "tail_one_by_one", "portions", "mixed")}
    eng, tensors = engine_and_weights(dtype, 1024, **(dict(tuning="auto", tune_min_bytes=1e6) if tuned else dict(tuning="measured")))
    if tuned:
        table = eng.tuning_table()
        assert len(table["tcgen05"]) >= 12 and len(table["slices"]) >= 9 and any(table["tcgen05"].values()), table
    else:
        assert not eng.tuning_table()["tcgen05"]
    rounding = "bfloat16" if dtype == "bfloat16" else None
    w = {k: v.to(torch.float64) for k, v in tensors.items()}
    # sharpen attention as the tiny tests do (scores of random weights are all near zero otherwise)
    for k in w:
        if k.endswith("q_norm.weight") or k.endswith("k_norm.weight"):
            w[k] = w[k] * 2.0
    for block in eng.spec.blocks:
        block.mixer.q_norm.mul_(2.0)
        block.mixer.k_norm.mul_(2.0)
    ref = {rid: plain.forward(SHAPE_8B, w, ids, rounding).float().cpu() for rid, ids in reqs.items()}
    tol = 2e-5 if dtype == "float32" else 2e-2
    scale = max(r.abs().max().item() for r in ref.values())
    results = {}
    for way, steps in steps_by_way.items():
        got = replay.run_engine(eng, steps)
        eng.pools.table.check()
        for rid in reqs:
            assert tiny.max_abs(got[rid], ref[rid]) < tol * max(1.0, scale), (way, rid)
        results[way] = got
    if dtype == "float32":
        for way in ("tail_one_by_one", "portions", "mixed"):
            for rid in reqs:
                assert torch.equal(results[way][rid], results["whole"][rid]), (way, rid)
    if tuned:
        import json
        del eng
        again, _ = engine_and_weights(dtype, 1024, tuning=json.loads(json.dumps(table)))
        for block in again.spec.blocks:
            block.mixer.q_norm.mul_(2.0)
            block.mixer.k_norm.mul_(2.0)
        assert again.tuning_table() == table
        got = replay.run_engine(again, steps_by_way["tail_one_by_one"])
        for rid in reqs:
            assert torch.equal(got[rid], results["tail_one_by_one"][rid]), rid
        # another engine in the same process knows nothing of it
        from rust_mlx_b200.kernels import ops
        assert not ops.default.tuned and not ops.Kernels("auto").tuned
