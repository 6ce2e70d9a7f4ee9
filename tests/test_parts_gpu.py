"""Each part of a layer alone, built from sizes only, against the plain implementation's
function of the same name; and a model whose schedule is not the plain one."""
import pytest
import torch

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
F = torch.float64


def context(dtype=torch.float32):
    from rust_mlx_b200.engine.workspace import Workspace
    from rust_mlx_b200.kernels import ops
    from rust_mlx_b200.parts import BuildContext
    return BuildContext(DEV, dtype, ops.default, Workspace(DEV))


def bind(part, seed=0, dtype=torch.float32):
    from rust_mlx_b200.weights.random_init import random_tensors
    tensors = random_tensors(part.all_param_specs(), seed, dtype, DEV)
    host = {k: v.detach().cpu().to(F) for k, v in tensors.items()}
    part.bind_all(tensors, context(dtype))
    return host


def test_rmsnorm_part():
    from rust_mlx_b200.parts.norm import RMSNorm
    norm = RMSNorm("n.weight", 200, 3e-4)
    w = bind(norm)
    h = torch.randn(9, 200, device=DEV)
    delta = torch.randn(9, 200, device=DEV)
    h0 = h.clone()
    h2, x = norm.forward(h, delta)
    assert h2 is h and torch.allclose(h, h0 + delta)
    want = plain.rms_norm((h0 + delta).double().cpu(), w["n.weight"], 3e-4)
    assert tiny.max_abs(x.cpu(), want) < 1e-5
    rows = torch.tensor([8, 2], dtype=torch.int32, device=DEV)
    xr = norm.forward_rows(h, None, rows)
    assert tiny.max_abs(xr.cpu(), want[[8, 2]]) < 1e-5


@pytest.mark.parametrize("inner", [200, 192])   # 192: gate and up rows fused in blocks of 64
def test_swiglu_part(inner):
    from rust_mlx_b200.parts.feedforward import SwiGLUFeedForward
    ff = SwiGLUFeedForward("mlp", 72, inner)
    w = bind(ff, seed=2)
    assert ff.block == (64 if inner % 64 == 0 else 0)
    x = torch.randn(11, 72, device=DEV)
    y = ff.forward(x)
    want = plain.swiglu_mlp(x.double().cpu(), {k.replace("mlp", "m"): v for k, v in w.items()}, "m", lambda t: t)
    assert tiny.max_abs(y.cpu(), want) < 1e-6


def test_swiglu_part_bfloat16_takes_the_fused_product():
    from rust_mlx_b200.kernels import ops
    from rust_mlx_b200.parts.feedforward import SwiGLUFeedForward
    ff = SwiGLUFeedForward("mlp", 256, 640)
    w = bind(ff, seed=3, dtype=torch.bfloat16)
    x = torch.randn(9, 256, device=DEV).to(torch.bfloat16)
    assert ops.prefers_fused_swiglu(9, 1280, 256)
    before = ops.launch_count
    y = ff.forward(x)
    assert ops.launch_count - before <= 2            # gate/up with SwiGLU in one kernel; no pointwise kernel
    r = lambda t: t.to(torch.bfloat16).double()
    want = plain.swiglu_mlp(x.double().cpu(), {k.replace("mlp", "m"): v for k, v in w.items()}, "m", r)
    assert ((y.double().cpu() - want).abs() <= 1e-2 * (1 + want.abs())).all()


def test_rotary_part_and_partial_rotation():
    from rust_mlx_b200.parts.position import NoPositionEncoding, RotaryEmbedding
    rope = RotaryEmbedding(48, 5000.0, rotary_dim=32)
    rope.bind({}, context())
    want = (5000.0 ** (-2.0 * torch.arange(16, dtype=F) / 32)).float()
    assert torch.equal(rope.inv_freq.cpu(), want)
    assert NoPositionEncoding().rotary_dim == 0
    with pytest.raises(ValueError):
        RotaryEmbedding(48, 5000.0, rotary_dim=50)


@pytest.mark.parametrize("window, qk_norm, rot", [(0, True, 24), (6, True, 24), (0, False, 12), (0, True, 0)])
def test_attention_part_over_two_steps(window, qk_norm, rot):
    """The mixer alone with a cache of its own: a prompt portion, then single tokens."""
    from rust_mlx_b200.cache import CachePools
    from rust_mlx_b200.engine.batch import SequenceInput, build_batch
    from rust_mlx_b200.parts.attention import AttentionMixer
    from rust_mlx_b200.parts.position import NoPositionEncoding, RotaryEmbedding
    width, nq, nkv, hd, page = 40, 6, 3, 24, 4
    pos_enc = RotaryEmbedding(hd, 777.0, rotary_dim=rot) if rot else NoPositionEncoding()
    mixer = AttentionMixer("a", width, nq, nkv, hd, pos_enc, qk_norm_eps=2e-5 if qk_norm else None, window=window)
    w = bind(mixer, seed=4)
    pools = CachePools({0: mixer.cache_spec()}, max_tokens=64, page_size=page, max_requests=2, dtype=torch.float32, device=DEV)
    T = 19
    x = torch.randn(T, width, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pools.open(7)
    outs, at = [], 0
    for c in (11, 1, 5, 1, 1):
        pools.table.reserve(7, at + c)
        batch = build_batch([SequenceInput(7, at, [0] * c, [])], pools, DEV, status, 10)
        outs.append(mixer.forward(x[at:at + c].contiguous(), batch, pools.view(0, batch, False)).clone())
        at += c
        pools.table.commit(7, at)
    got = torch.cat(outs).cpu()
    assert status.item() == 0
    # the plain implementation, part by part
    xd = x.double().cpu()
    pos = torch.arange(T)
    q = plain.linear(xd, w["a.q_proj.weight"]).reshape(T, nq, hd)
    k = plain.linear(xd, w["a.k_proj.weight"]).reshape(T, nkv, hd)
    v = plain.linear(xd, w["a.v_proj.weight"]).reshape(T, nkv, hd)
    if qk_norm:
        q, k = plain.rms_norm(q, w["a.q_norm.weight"], 2e-5), plain.rms_norm(k, w["a.k_norm.weight"], 2e-5)
    if rot:
        q, k = plain.rope(q, pos, 777.0, rot), plain.rope(k, pos, 777.0, rot)
    o = plain.attention_scores(q, k, v, pos, window)
    want = plain.linear(o.reshape(T, nq * hd), w["a.o_proj.weight"])
    assert tiny.max_abs(got, want) < 1e-5


def test_block_part():
    from rust_mlx_b200.cache import CachePools
    from rust_mlx_b200.engine.batch import SequenceInput, build_batch
    from rust_mlx_b200.parts.attention import AttentionMixer
    from rust_mlx_b200.parts.block import PreNormBlock
    from rust_mlx_b200.parts.feedforward import SwiGLUFeedForward
    from rust_mlx_b200.parts.norm import RMSNorm
    from rust_mlx_b200.parts.position import RotaryEmbedding
    width, nq, nkv, hd = 48, 4, 1, 16
    block = PreNormBlock(RMSNorm("n1", width, 1e-5), AttentionMixer("a", width, nq, nkv, hd, RotaryEmbedding(hd, 100.0), 1e-5),
                         RMSNorm("n2", width, 1e-5), SwiGLUFeedForward("m", width, 80))
    w = bind(block, seed=6)
    pools = CachePools({0: block.mixer.cache_spec()}, max_tokens=32, page_size=8, max_requests=1, dtype=torch.float32, device=DEV)
    pools.open(0)
    pools.table.reserve(0, 13)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = build_batch([SequenceInput(0, 0, [0] * 13, [])], pools, DEV, status, 10)
    h = torch.randn(13, width, device=DEV)
    pending = torch.randn(13, width, device=DEV)
    hd0 = (h + pending).double().cpu()
    h2, m = block.forward(h, pending, batch, pools.view(0, batch, False))
    config = dict(num_attention_heads=nq, num_key_value_heads=nkv, head_dim=hd, rms_norm_eps=1e-5, rope_theta=100.0)
    wp = {("L.self_attn." + k[2:] if k.startswith("a.") else "L.mlp." + k[2:] if k.startswith("m.") else k): v
          for k, v in w.items()}
    x = plain.rms_norm(hd0, w["n1"], 1e-5)
    h1 = hd0 + plain.attention(x, wp, "L.self_attn", config, torch.arange(13), 0, lambda t: t)
    want_m = plain.swiglu_mlp(plain.rms_norm(h1, w["n2"], 1e-5), wp, "L.mlp", lambda t: t)
    assert tiny.max_abs(h2.cpu(), h1) < 1e-5 and tiny.max_abs(m.cpu(), want_m) < 1e-5


def test_embedding_and_heads():
    from rust_mlx_b200.parts.embedding import OutputHead, TokenEmbedding
    from rust_mlx_b200.parts.base import Part
    emb = TokenEmbedding("e", 77, 24)
    tied, own = OutputHead(77, 24, tied_to=emb), OutputHead(77, 24, name="head")

    class Both(Part):
        def children(self):
            return [emb, tied, own]
    w = bind(Both(), seed=8)
    ids = torch.tensor([3, 76, 0, 3], dtype=torch.int32, device=DEV)
    assert tiny.max_abs(emb.forward(ids).cpu(), w["e"][[3, 76, 0, 3]]) == 0
    x = torch.randn(5, 24, device=DEV)
    assert tiny.max_abs(tied.forward(x).clone().cpu(), x.double().cpu() @ w["e"].t()) < 1e-5
    assert tiny.max_abs(own.forward(x).clone().cpu(), x.double().cpu() @ w["head"].t()) < 1e-5
    with pytest.raises(ValueError):
        OutputHead(77, 24)


def test_schedule_is_data_a_layer_twice_and_a_shared_cache(tmp_path):
    """A model that runs layer 1 twice and lets the second run read the first run's cache:
    registered here, built by the engine from config.json, compared with the plain functions."""
    import json
    from rust_mlx_b200.config import Qwen3Config
    from rust_mlx_b200.engine import Engine
    from rust_mlx_b200.models.qwen3 import build_qwen3
    from rust_mlx_b200.parts import LayerCall
    from rust_mlx_b200.registry import register_architecture, unregister_architecture
    from rust_mlx_b200.weights import write_random_model

    def build(config):
        spec = build_qwen3(config)
        spec.schedule = [LayerCall(0, 0), LayerCall(1, 1), LayerCall(1, 1), LayerCall(0, 2)]
        spec.check_schedule()
        return spec

    register_architecture("TwiceForCausalLM", Qwen3Config, build)
    try:
        raw = dict(tiny.TINY_A, architectures=["TwiceForCausalLM"])
        folder = str(tmp_path / "twice")
        write_random_model(Qwen3Config.from_dict(raw), folder, seed=9, store_dtype="float32")
        folder = tiny.sharpen(folder)
        eng = Engine(folder, dtype="float32", max_tokens=64, page_size=16, max_requests=2)
        assert len(eng.pools.groups) == 1 and len(eng.pools.groups[0].cache_ids) == 3
        ids = tiny.prompts(256, [21], seed=1)[0]
        got = torch.cat([eng.step([("a", ids[:13], list(range(13)))]), eng.step([("a", ids[13:], list(range(8)))])]).cpu()
    finally:
        unregister_architecture("TwiceForCausalLM")
    config, tensors = plain.read_folder(folder)
    w = plain.prepare_weights(config, tensors, None)
    T, pos, eps = len(ids), torch.arange(len(ids)), config["rms_norm_eps"]
    nq, nkv, hd = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    ident = lambda t: t
    h = plain.embedding(w["model.embed_tokens.weight"], ids)
    kept = {}
    for layer, cache, writes in ((0, 0, True), (1, 1, True), (1, 1, False), (0, 2, True)):
        p = f"model.layers.{layer}"
        x = plain.rms_norm(h, w[p + ".input_layernorm.weight"], eps)
        a = p + ".self_attn"
        q = plain.rope(plain.rms_norm(plain.linear(x, w[a + ".q_proj.weight"]).reshape(T, nq, hd), w[a + ".q_norm.weight"], eps),
                       pos, config["rope_theta"], hd)
        if writes:
            k = plain.rope(plain.rms_norm(plain.linear(x, w[a + ".k_proj.weight"]).reshape(T, nkv, hd), w[a + ".k_norm.weight"], eps),
                           pos, config["rope_theta"], hd)
            kept[cache] = (k, plain.linear(x, w[a + ".v_proj.weight"]).reshape(T, nkv, hd))
        k, v = kept[cache]
        o = plain.attention_scores(q, k, v, pos, 0)
        h = h + plain.linear(o.reshape(T, nq * hd), w[a + ".o_proj.weight"])
        h = h + plain.swiglu_mlp(plain.rms_norm(h, w[p + ".post_attention_layernorm.weight"], eps), w, p + ".mlp", ident)
    want = plain.linear(plain.rms_norm(h, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])
    assert tiny.max_abs(got, want) < 2e-5
