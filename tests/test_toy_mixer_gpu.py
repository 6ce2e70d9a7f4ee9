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
        # generation through the scheduler works for it too: the scheduler takes slots from the page table itself,
        # and a request it admits (or admits again after it stepped back) must not see what the slot's last owner
        # left there: the slots are made dirty first, and the short prompts would show it
        def follows_plain(prompts, out):
            for p, toks in zip(prompts, out):
                ids = list(p)
                for t in toks:
                    logits = plain_toy_logits(folder, ids)[-1]
                    assert logits[t] >= logits.max() - 1e-5, (len(p), len(ids))
                    ids.append(t)
        for grp in eng.pools.state_groups:
            grp.state.fill_(50.0)
        ps = [reqs["r3"], reqs["r0"], reqs["r1"]]
        follows_plain(ps, eng.generate(ps, max_tokens=5, prefill_chunk=4))
        small = Engine(folder, dtype="float32", max_tokens=80, page_size=8, max_requests=3)   # ten pages: not enough
        for grp in small.pools.state_groups:
            grp.state.fill_(-30.0)
        ps = [reqs["r1"], reqs["r4"], reqs["r2"]]
        r = small.generate_detailed(ps, max_tokens=12, prefill_chunk=8, ignore_eos=True)
        assert r.preemptions > 0
        follows_plain(ps, r.tokens)
        assert small.pools.table.live() == 0
    finally:
        unregister_architecture("ToyStateForCausalLM")


def test_toy_routed_feed_forward_and_unrotated_layers(tmp_path):
    """Two more toy parts defined here and built by the engine without a change to its files: a feed-forward
    that routes every token to its best expert of three (router logits and the choice in float32, so the
    choice does not depend on the batch), and attention layers without any position encoding.  Stepped in
    portions and mixed batches, compared with the plain restatement below."""
    import replay
    from rust_mlx_b200.config import Qwen3Config
    from rust_mlx_b200.engine import Engine
    from rust_mlx_b200.models.qwen3 import build_qwen3
    from rust_mlx_b200.parts import FeedForward, ParamSpec
    from rust_mlx_b200.parts.position import NoPositionEncoding
    from rust_mlx_b200.registry import register_architecture, unregister_architecture
    from rust_mlx_b200.weights import write_random_model

    class RoutedFeedForward(FeedForward):
        def __init__(self, prefix, width, inner, experts):
            self.prefix, self.width, self.inner, self.experts = prefix, width, inner, experts

        def param_specs(self):
            p = self.prefix
            specs = [ParamSpec(f"{p}.router.weight", (self.experts, self.width), "linear", "float32")]
            for e in range(self.experts):
                specs += [ParamSpec(f"{p}.experts.{e}.up.weight", (self.inner, self.width)),
                          ParamSpec(f"{p}.experts.{e}.down.weight", (self.width, self.inner))]
            return specs

        def bind(self, tensors, ctx):
            super().bind(tensors, ctx)
            p = self.prefix
            self.router = tensors[f"{p}.router.weight"]
            self.up = [tensors[f"{p}.experts.{e}.up.weight"] for e in range(self.experts)]
            self.down = [tensors[f"{p}.experts.{e}.down.weight"] for e in range(self.experts)]

        def forward(self, x, batch=None):
            logits = x.float() @ self.router.t()
            choice = logits.argmax(-1)
            weight = torch.softmax(logits, -1).gather(1, choice[:, None])
            y = torch.zeros_like(x)
            for e in range(self.experts):
                rows = (choice == e).nonzero()[:, 0]
                if rows.numel():
                    h = torch.relu(x[rows].float() @ self.up[e].float().t())
                    y[rows] = ((h @ self.down[e].float().t()) * weight[rows]).to(x.dtype)
            return y

    def build(config):
        spec = build_qwen3(config)
        for i, block in enumerate(spec.blocks):
            block.ffn = RoutedFeedForward(f"model.layers.{i}.moe", config.hidden_size, config.intermediate_size, 3)
            if i % 2 == 1:
                block.mixer.position = NoPositionEncoding()
        return spec

    def plain_logits(folder, ids):
        config, tensors = plain.read_folder(folder)
        w = plain.prepare_weights(config, tensors, None)
        eps, T = config["rms_norm_eps"], len(ids)
        nq, nkv, hd = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
        pos = torch.arange(T)
        h = plain.embedding(w["model.embed_tokens.weight"], ids)
        for i in range(config["num_hidden_layers"]):
            p = f"model.layers.{i}"
            x = plain.rms_norm(h, w[p + ".input_layernorm.weight"], eps)
            a = p + ".self_attn"
            q = plain.rms_norm(plain.linear(x, w[a + ".q_proj.weight"]).reshape(T, nq, hd), w[a + ".q_norm.weight"], eps)
            k = plain.rms_norm(plain.linear(x, w[a + ".k_proj.weight"]).reshape(T, nkv, hd), w[a + ".k_norm.weight"], eps)
            v = plain.linear(x, w[a + ".v_proj.weight"]).reshape(T, nkv, hd)
            if i % 2 == 0:
                q, k = plain.rope(q, pos, config["rope_theta"], hd), plain.rope(k, pos, config["rope_theta"], hd)
            o = plain.attention_scores(q, k, v, pos, 0)
            h = h + plain.linear(o.reshape(T, nq * hd), w[a + ".o_proj.weight"])
            x = plain.rms_norm(h, w[p + ".post_attention_layernorm.weight"], eps)
            logits = x.float().double() @ w[p + ".moe.router.weight"].t()
            choice = logits.float().argmax(-1)
            weight = torch.softmax(logits, -1).gather(1, choice[:, None])
            y = torch.zeros_like(x)
            for e in range(3):
                rows = (choice == e).nonzero()[:, 0]
                if rows.numel():
                    hid = torch.relu(x[rows] @ w[f"{p}.moe.experts.{e}.up.weight"].t())
                    y[rows] = (hid @ w[f"{p}.moe.experts.{e}.down.weight"].t()) * weight[rows]
            h = h + y
        return plain.linear(plain.rms_norm(h, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])

    register_architecture("ToyRoutedForCausalLM", Qwen3Config, build)
    try:
        raw = dict(tiny.TINY_A, architectures=["ToyRoutedForCausalLM"])
        folder = str(tmp_path / "routed")
        write_random_model(Qwen3Config.from_dict(raw), folder, seed=31, store_dtype="float32")
        names = set(plain.read_folder(folder)[1])
        assert "model.layers.0.moe.router.weight" in names and "model.layers.0.mlp.gate_proj.weight" not in names
        reqs = {f"r{i}": p for i, p in enumerate(tiny.prompts(256, [19, 6, 33, 12], seed=2))}
        ref = {rid: plain_logits(folder, ids).float() for rid, ids in reqs.items()}
        for way in ("whole", "portions", "mixed"):
            steps = getattr(replay, way)(reqs, **({"live": 3} if way == "mixed" else {}))
            eng = Engine(folder, dtype="float32", max_tokens=replay.tokens_needed(steps, 16), page_size=16, max_requests=3)
            assert eng.graphs is None      # the toy part does not declare itself safe to capture
            got = replay.run_engine(eng, steps)
            for rid in reqs:
                assert tiny.max_abs(got[rid], ref[rid]) < 5e-5, (way, rid)
    finally:
        unregister_architecture("ToyRoutedForCausalLM")


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("D", "bfloat16")])
def test_toy_position_encoding(tmp_path, name, dtype):
    """Another position encoding, defined here and built by the engine without a change to its files: the angle of
    pair j at position p is ln(1 + p) (j + 1) 0.37, which no table of inverse frequencies expresses (it is not a
    multiple of the position), over the first three quarters of a head only, and with a factor of its own on the
    scores.  The mixer asks its position encoding for the step's cosines and sines and hands them to the kernels
    (in bfloat16 with heads of 128 a decoding step's attention kernel rotates with them itself).  Whole, in
    portions, token by token at the end, and mixed; compared with the plain restatement below."""
    import replay
    from rust_mlx_b200.config import Qwen3Config
    from rust_mlx_b200.engine import Engine
    from rust_mlx_b200.models.qwen3 import build_qwen3
    from rust_mlx_b200.parts import PositionEncoding
    from rust_mlx_b200.parts.attention import AttentionMixer
    from rust_mlx_b200.registry import register_architecture, unregister_architecture
    from rust_mlx_b200.weights import write_random_model

    def toy_angles(positions, rotary_dim):
        j = torch.arange(rotary_dim // 2, device=positions.device, dtype=torch.float32)
        return torch.log1p(positions.to(torch.float32))[:, None] * ((j + 1.0) * 0.37)

    class LogPositions(PositionEncoding):
        score_scale = 1.25

        def __init__(self, rotary_dim):
            self.rotary_dim, self.inv_freq = rotary_dim, None

        def angles(self, batch):
            key = ("log positions", self.rotary_dim)
            if key not in batch.per_step:
                a = toy_angles(batch.positions, self.rotary_dim)
                batch.per_step[key] = torch.cat([a.cos(), a.sin()], 1).contiguous()
            return batch.per_step[key]

    raw, page = tiny.CONFIGS[name]
    rotary = raw["head_dim"] if dtype == "bfloat16" else raw["head_dim"] * 3 // 4 // 2 * 2

    def build(config):
        spec = build_qwen3(config)
        toy = LogPositions(rotary)
        for block in spec.blocks:
            old = block.mixer
            block.mixer = AttentionMixer(old.prefix, old.width, old.heads, old.kv_heads, old.head_dim, toy,
                                         qk_norm_eps=old.qk_norm_eps, window=old.window, bias=old.bias)
        return spec

    def rotate(x, positions):   # half-split pairs (j, j + rotary / 2) of the first `rotary` numbers of every head
        a = toy_angles(positions, rotary).double()[:, None, :]
        half = rotary // 2
        x1, x2 = x[..., :half], x[..., half:rotary]
        return torch.cat([x1 * a.cos() - x2 * a.sin(), x2 * a.cos() + x1 * a.sin(), x[..., rotary:]], -1)

    def plain_logits(folder, ids, rounding=None):
        """The plain implementation's forward pass (tests/plain_qwen3.py: ``forward``, ``attention``) with the toy
        rotation and the factor on the scores in place of the model's own."""
        config, tensors = plain.read_folder(folder)
        w = plain.prepare_weights(config, tensors, rounding)
        r = plain.make_round(rounding)
        eps, T = config["rms_norm_eps"], len(ids)
        nq, nkv, hd = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
        pos = torch.arange(T)
        windows = plain.layer_windows(config)
        h = plain.embedding(w["model.embed_tokens.weight"], ids)
        for i in range(config["num_hidden_layers"]):
            p = f"model.layers.{i}"
            a = p + ".self_attn"
            x = r(plain.rms_norm(h, w[p + ".input_layernorm.weight"], eps))
            q = plain.linear(x, w[a + ".q_proj.weight"], None, r).reshape(T, nq, hd)
            k = plain.linear(x, w[a + ".k_proj.weight"], None, r).reshape(T, nkv, hd)
            v = plain.linear(x, w[a + ".v_proj.weight"], None, r).reshape(T, nkv, hd)
            q = r(rotate(plain.rms_norm(q, w[a + ".q_norm.weight"], eps), pos))
            k = r(rotate(plain.rms_norm(k, w[a + ".k_norm.weight"], eps), pos))
            o = r(plain.attention_scores(q, k, v, pos, windows[i], 1.25))
            h = h + plain.linear(o.reshape(T, nq * hd), w[a + ".o_proj.weight"], None, r)
            x = r(plain.rms_norm(h, w[p + ".post_attention_layernorm.weight"], eps))
            h = h + plain.swiglu_mlp(x, w, p + ".mlp", r)
        x = r(plain.rms_norm(h, w["model.norm.weight"], eps))
        head = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings") else w["lm_head.weight"]
        return plain.linear(x, head)

    register_architecture("ToyLogPositionsForCausalLM", Qwen3Config, build)
    try:
        config = dict(raw, architectures=["ToyLogPositionsForCausalLM"])
        folder = str(tmp_path / "logpos")
        write_random_model(Qwen3Config.from_dict(config), folder, seed=37, store_dtype="float32" if dtype == "float32" else "bfloat16")
        reqs = {f"r{i}": p for i, p in enumerate(tiny.prompts(raw["vocab_size"], [70, 41, 9, 55], seed=6))}
        exact = {rid: plain_logits(folder, ids).float() for rid, ids in reqs.items()}
        bound = {rid: 5e-5 for rid in reqs}
        if dtype == "bfloat16":   # as far from the exact logits as the same roundings put the plain restatement, at least 2e-2
            bound = {rid: max(2e-2, tiny.max_abs(plain_logits(folder, ids, "bfloat16").float(), exact[rid])) for rid, ids in reqs.items()}
        for way in ("whole", "portions", "tail_one_by_one", "mixed"):
            steps = getattr(replay, way)(reqs, **({"live": 3} if way == "mixed" else {}))
            eng = Engine(folder, dtype=dtype, max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
            assert eng.graphs is None      # the toy part does not declare itself safe to capture
            got = replay.run_engine(eng, steps)
            for rid in reqs:
                assert tiny.max_abs(got[rid], exact[rid]) < bound[rid], (way, rid, tiny.max_abs(got[rid], exact[rid]))
    finally:
        unregister_architecture("ToyLogPositionsForCausalLM")


def test_toy_block_that_remembers_two_things(tmp_path):
    """A block defined here with two stateful sub-layers (attention over pages and a running average in a state
    slot, side by side): it says so in ``cache_specs()``, its schedule entry names one cache id for each, and its
    ``forward`` gets a tuple of views.  Built, stepped (whole, in portions, mixed) and generated from without a
    change to the framework's files."""
    import replay
    from rust_mlx_b200.config import Qwen3Config
    from rust_mlx_b200.engine import Engine
    from rust_mlx_b200.models.qwen3 import build_qwen3
    from rust_mlx_b200.parts import LayerCall, Part
    from rust_mlx_b200.registry import register_architecture, unregister_architecture
    from rust_mlx_b200.weights import write_random_model
    Toy = make_toy()

    class TwoMemoryBlock(Part):
        def __init__(self, inner, toy):
            self.inner, self.toy = inner, toy          # a pre-norm block of the framework and the second sub-layer

        def children(self):
            return [self.inner, self.toy]

        def cache_specs(self):
            return self.inner.cache_specs() + self.toy.cache_specs()

        def forward(self, h, pending, batch, cache):
            pages, slots = cache
            b = self.inner
            h, x = b.norm1.forward(h, pending)
            a = b.mixer.forward(x, batch, pages) + self.toy.forward(x, batch, slots)
            h, x = b.norm2.forward(h, a)
            return h, b.ffn.forward(x, batch)

    def build(config):
        spec = build_qwen3(config)
        for i in (0, 2):
            spec.blocks[i] = TwoMemoryBlock(spec.blocks[i], Toy(f"model.layers.{i}.toy", config.hidden_size, 0.6))
        spec.schedule = [LayerCall(0, (0, 10)), LayerCall(1, 1), LayerCall(2, (2, 12))]
        spec.check_schedule()
        return spec

    def plain_logits(folder, ids):
        config, tensors = plain.read_folder(folder)
        w = plain.prepare_weights(config, tensors, None)
        eps, T = config["rms_norm_eps"], len(ids)
        h = plain.embedding(w["model.embed_tokens.weight"], ids)
        for i in range(3):
            p = f"model.layers.{i}"
            x = plain.rms_norm(h, w[p + ".input_layernorm.weight"], eps)
            h = h + plain.attention(x, w, p + ".self_attn", config, torch.arange(T), 0, lambda t: t)
            if i in (0, 2):
                s, rows = torch.zeros(config["hidden_size"], dtype=torch.float64), []
                for t in range(T):
                    s = 0.6 * s + x[t]
                    rows.append(s @ w[p + ".toy.mix.weight"].t())
                h = h + torch.stack(rows)
            h = h + plain.swiglu_mlp(plain.rms_norm(h, w[p + ".post_attention_layernorm.weight"], eps), w, p + ".mlp", lambda t: t)
        return plain.linear(plain.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"])

    register_architecture("ToyTwoMemoriesForCausalLM", Qwen3Config, build)
    try:
        raw = dict(tiny.TINY_B, architectures=["ToyTwoMemoriesForCausalLM"])
        folder = str(tmp_path / "two")
        write_random_model(Qwen3Config.from_dict(raw), folder, seed=5, store_dtype="float32")
        reqs = {f"r{i}": p for i, p in enumerate(tiny.prompts(509, [12, 31, 5, 20], seed=8))}
        ref = {rid: plain_logits(folder, ids).float() for rid, ids in reqs.items()}
        for way in ("whole", "portions", "mixed"):
            steps = getattr(replay, way)(reqs, **({"live": 3} if way == "mixed" else {}))
            eng = Engine(folder, dtype="float32", max_tokens=replay.tokens_needed(steps, 8), page_size=8, max_requests=3)
            assert sorted(g.spec.kind for g in eng.pools.groups) == ["paged", "state"]
            assert len(eng.pools.paged_groups[0].cache_ids) == 3 and len(eng.pools.state_groups[0].cache_ids) == 2
            got = replay.run_engine(eng, steps)
            for rid in reqs:
                assert tiny.max_abs(got[rid], ref[rid]) < 2e-5, (way, rid)
        for grp in eng.pools.state_groups:
            grp.state.fill_(9.0)
        out = eng.generate([reqs["r2"], reqs["r0"]], max_tokens=4, prefill_chunk=5)
        for p, toks in zip([reqs["r2"], reqs["r0"]], out):
            ids = list(p)
            for t in toks:
                logits = plain_logits(folder, ids)[-1]
                assert logits[t] >= logits.max() - 1e-5
                ids.append(t)
        # a schedule entry that names the wrong number of caches is refused when the model is built
        with pytest.raises(ValueError, match="remembers 2"):
            spec = build(Qwen3Config.from_dict(raw))
            spec.schedule[0] = LayerCall(0, 0)
            spec.check_schedule()
    finally:
        unregister_architecture("ToyTwoMemoriesForCausalLM")
