"""A toy mixer with state of its own, defined here, is registered, built and stepped
without a change to the framework's files.

The mixer keeps a running average per request, s <- decay * s + x_t, y_t = s . W^T, in a
state slot of fixed size (no pages).  A model alternates it with attention layers, so the
cache manager holds a paged group and a state group side by side.  The toy's arithmetic
uses torch operations: it stands for "a part someone else wrote", not for a product kernel.
"""
import json
import os

import pytest
import torch

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu


def make_toy():
    from rust_mlx_b200.parts import CacheSpec, Mixer, ParamSpec

    class RunningAverageMixer(Mixer):
        def __init__(self, prefix, width, decay):
            self.prefix, self.width, self.decay = prefix, width, decay

        def cache_spec(self):
            return CacheSpec("state", state_shape=(self.width,), state_dtype="float32")

        def param_specs(self):
            return [ParamSpec(f"{self.prefix}.mix.weight", (self.width, self.width))]

        def bind(self, tensors, ctx):
            super().bind(tensors, ctx)
            self.weight = tensors[f"{self.prefix}.mix.weight"]

        def forward(self, x, batch, cache):
            out = torch.empty_like(x)
            for i, slot in enumerate(cache.slots_host):           # sequences of the batch, each in order
                a, b = batch.q_start_host[i], batch.q_start_host[i + 1]
                s = cache.state[slot]
                for t in range(a, b):
                    s = self.decay * s + x[t].float()
                    out[t] = (s @ self.weight.float().t()).to(x.dtype)
                if not cache.read_only:
                    cache.state[slot] = s
            return out

    return RunningAverageMixer


def build_toy_model(config):
    from rust_mlx_b200.models.qwen3 import build_qwen3
    Toy = make_toy()
    spec = build_qwen3(config)
    for i, block in enumerate(spec.blocks):
        if i % 2 == 1:
            block.mixer = Toy(f"model.layers.{i}.toy", config.hidden_size, 0.5 + 0.1 * i)
    spec.check_schedule()
    return spec


def plain_toy_logits(folder, ids):
    config, tensors = plain.read_folder(folder)
    w = plain.prepare_weights(config, tensors, None)
    eps, T = config["rms_norm_eps"], len(ids)
    h = plain.embedding(w["model.embed_tokens.weight"], ids)
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}"
        x = plain.rms_norm(h, w[p + ".input_layernorm.weight"], eps)
        if i % 2 == 1:
            s = torch.zeros(config["hidden_size"], dtype=torch.float64)
            rows = []
            for t in range(T):
                s = (0.5 + 0.1 * i) * s + x[t]
                rows.append(s @ w[p + ".toy.mix.weight"].t())
            h = h + torch.stack(rows)
        else:
            h = h + plain.attention(x, w, p + ".self_attn", config, torch.arange(T), 0, lambda t: t)
        h = h + plain.swiglu_mlp(plain.rms_norm(h, w[p + ".post_attention_layernorm.weight"], eps), w, p + ".mlp", lambda t: t)
    return plain.linear(plain.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"])


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from rust_mlx_b200.config import Qwen3Config
    from rust_mlx_b200.engine import Engine
    from rust_mlx_b200.registry import register_architecture, unregister_architecture
    from rust_mlx_b200.weights import write_random_model
    import replay

    register_architecture("ToyStateForCausalLM", Qwen3Config, build_toy_model)
    try:
        raw = dict(tiny.TINY_B, architectures=["ToyStateForCausalLM"], use_sliding_window=False, num_hidden_layers=4)
        folder = str(tmp_path / "toy")
        write_random_model(Qwen3Config.from_dict(raw), folder, seed=21, store_dtype="float32")
        names = set(plain.read_folder(folder)[1])
        assert "model.layers.1.toy.mix.weight" in names and "model.layers.1.self_attn.q_proj.weight" not in names
        reqs = {f"r{i}": p for i, p in enumerate(tiny.prompts(509, [9, 30, 17, 4, 26], seed=3))}
        ref = {rid: plain_toy_logits(folder, ids).float() for rid, ids in reqs.items()}
        steps = replay.mixed(reqs, live=3)
        eng = Engine(folder, dtype="float32", max_tokens=replay.tokens_needed(steps, 8), page_size=8, max_requests=3)
        kinds = sorted(g.spec.kind for g in eng.pools.groups)
        assert kinds == ["paged", "state"]
        got = replay.run_engine(eng, steps)
        for rid in reqs:
            assert tiny.max_abs(got[rid], ref[rid]) < 2e-5, rid
        # slots were used again by later requests, and a new request starts from zero state
        assert eng.pools.table.live() == 0 and eng.pools.table.free_slots() == 3
        whole = replay.run_engine(eng, replay.whole(reqs))
        for rid in reqs:
            assert tiny.max_abs(whole[rid], ref[rid]) < 2e-5, rid
        # generation through the scheduler works for it too
        out = eng.generate([reqs["r0"], reqs["r1"]], max_tokens=5, prefill_chunk=4)
        ids = list(reqs["r1"])
        for t in out[1]:
            logits = plain_toy_logits(folder, ids)[-1]
            assert logits[t] >= logits.max() - 1e-5
            ids.append(t)
    finally:
        unregister_architecture("ToyStateForCausalLM")
