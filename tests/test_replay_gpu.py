"""Replay of the same requests cut in different ways, against the plain implementation.

Both tiny configurations, float32 and bfloat16.  The model folders are sharpened
(tiny.sharpen) so that a wrong, stale or missing key changes the logits by far more
than the tolerance.  Tolerances, fixed before the first run: float32 2e-5 (logits are
of order 1; sums of at most a few hundred float32 products), bfloat16 2e-2 against the
plain implementation restated with bfloat16 roundings (a flipped last bit of a
bfloat16 activation is 4e-3 of its value).  In float32 the four ways must agree bit
for bit: every kernel of that path adds in an order that depends on the position only.

The bfloat16 bound of a request is 2e-2, or the distance of the bfloat16 restatement itself
from the exact (float64) logits of that request where that is more: two bfloat16
evaluations of the same formulas that round at the same places still differ by flipped
last bits (sums are added in another order), and cannot be asked to agree better than
either agrees with the exact values.  (Met with B, full attention in all three layers,
sharpened: one request's restatement lies 0.0233 from its exact logits and the engine
0.0222 from the restatement; the named intermediates of that step agree bit for bit
through the first layer's norm and rotation and then differ by single last bits, 2^-6 at
values between 2 and 4.  A wrong, stale or missing key moves these logits by 0.5.)
"""
import os

import pytest
import torch

import plain_qwen3 as plain
import replay
import tiny

pytestmark = pytest.mark.gpu
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
LENGTHS = [5, 17, 33, 150, 41, 9, 64, 65]


@pytest.fixture(scope="module")
def workdir(tmp_path_factory):
    return tmp_path_factory.mktemp("replay")


def setup(workdir, name, dtype):
    raw, page = tiny.CONFIGS[name]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=3, store="float32"))
    reqs = {f"r{i}": p for i, p in enumerate(tiny.prompts(raw["vocab_size"], LENGTHS, seed=7))}
    pm = plain.PlainModel(folder, rounding=None if dtype == "float32" else "bfloat16")
    ref = {rid: pm.logits(t).float() for rid, t in reqs.items()}
    if dtype == "bfloat16":
        exact = plain.PlainModel(folder)
        for rid, t in reqs.items():
            _bound[(name, dtype, rid)] = max(TOL[dtype], tiny.max_abs(ref[rid], exact.logits(t).float()))
    return raw, page, folder, reqs, ref


_bound = {}


def bound_of(name, dtype, rid):
    return _bound.get((name, dtype, rid), TOL[dtype])


_cache = {}


def cached_setup(workdir, name, dtype):
    key = (name, dtype)
    if key not in _cache:
        _cache[key] = setup(workdir, name, dtype)
    return _cache[key]


def engine_for(folder, dtype, page, tokens):
    from rust_mlx_b200.engine import Engine
    return Engine(folder, dtype=dtype, max_tokens=tokens, page_size=page, max_requests=4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "Bw", "C", "D", "F", "G"])
@pytest.mark.parametrize("way", ["whole", "tail_one_by_one", "portions", "mixed"])
def test_every_way_of_cutting_matches_the_plain_implementation(workdir, name, dtype, way):
    raw, page, folder, reqs, ref = cached_setup(workdir, name, dtype)
    steps = getattr(replay, way)(reqs)
    need = replay.tokens_needed(steps, page)
    eng = engine_for(folder, dtype, page, need)   # exactly what the trace needs: pages are used again
    got = replay.run_engine(eng, steps)
    eng.pools.table.check()
    assert eng.pools.table.live() == 0 and eng.pools.table.free_pages(0) == eng.pools.num_pages
    for rid in reqs:
        assert got[rid].shape == ref[rid].shape
        assert tiny.max_abs(got[rid], ref[rid]) < bound_of(name, dtype, rid), (rid, way)
    _cache[(name, dtype, way)] = got


@pytest.mark.parametrize("name", ["A", "B", "Bw", "C", "D", "E", "F", "G"])
def test_float32_ways_agree_bit_for_bit(workdir, name):
    raw, page, folder, reqs, ref = cached_setup(workdir, name, "float32")
    results = []
    for way in ("whole", "tail_one_by_one", "portions", "mixed"):
        got = _cache.get((name, "float32", way))
        if got is None:
            steps = getattr(replay, way)(reqs)
            got = replay.run_engine(engine_for(folder, "float32", page, replay.tokens_needed(steps, page)), steps)
        results.append(got)
    for other in results[1:]:
        for rid in reqs:
            assert torch.equal(other[rid], results[0][rid])


LONG = [700, 333, 1100, 64, 257, 5]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name, seed", [("C", 1), ("C", 2), ("D", 3), ("B", 4), ("Bw", 7), ("E", 5), ("E", 6)])
def test_random_cuts_of_long_requests(workdir, name, seed, dtype):
    """Requests of up to 1,100 tokens (many key tiles, block tables of dozens of pages) cut at random: single
    tokens, small portions and portions of some hundred tokens of up to four requests in a step, a request
    now and then left out, in a cache that holds no more than the trace needs.

    The bound in bfloat16: over sequences this long the plain implementation restated with bfloat16 roundings
    lies 0.04 to 0.08 from the exact logits itself (measured here, per request), so two bfloat16 evaluations
    of the same formulas cannot be asked to agree to 2e-2 in every one of half a million logits: the engine
    must be as close to the restatement as the restatement is to the exact values (and to 2e-2 where that is
    more).  A wrong, stale or missing key moves logits by 0.5 and more (the weights are sharpened).

    In float32 the random cuts must give the bits that each request gives alone and whole; against the plain
    implementation (float64) the bound is 1e-4 here: reductions over up to 1,100 keys and three layers of them
    (unit roundoff 6e-8, times the square root of the terms, times some thirty reductions in a row, times what
    sharpened weights and norms amplify), where a product in reduced precision would show as 1e-3."""
    raw, page = tiny.CONFIGS[name]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=30 + seed, store="float32"))
    reqs = {f"q{i}": p for i, p in enumerate(tiny.prompts(raw["vocab_size"], LONG, seed=seed))}
    pm = plain.PlainModel(folder, rounding=None if dtype == "float32" else "bfloat16")
    exact = plain.PlainModel(folder)
    steps = replay.random_cuts(reqs, seed)
    assert max(len(e["tokens"]) for s in steps for e in s["entries"]) > 128 and max(len(s["entries"]) for s in steps) >= 3
    eng = engine_for(folder, dtype, page, replay.tokens_needed(steps, page))
    got = replay.run_engine(eng, steps)
    eng.pools.table.check()
    assert eng.pools.table.live() == 0
    if dtype == "float32":
        alone = replay.run_engine(engine_for(folder, dtype, page, max(-(-n // page) * page for n in LONG)), replay.whole(reqs))
        for rid in reqs:
            assert torch.equal(got[rid], alone[rid]), rid
    for rid, toks in reqs.items():
        want = pm.logits(toks)
        bound = 1e-4 if dtype == "float32" else max(TOL[dtype], tiny.max_abs(want.float(), exact.logits(toks).float()))
        assert tiny.max_abs(got[rid], want.float()) < bound, (rid, len(toks), bound)


@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_replay_uses_pages_again(workdir, name):
    raw, page, folder, reqs, ref = cached_setup(workdir, name, "float32")
    steps = replay.mixed(reqs)
    eng = engine_for(folder, "float32", page, replay.tokens_needed(steps, page))
    seen, again = {}, 0
    for s in steps:
        eng.step([(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        for e in s["entries"]:
            rid = eng._req_ids[e["id"]]
            for p in eng.pools.table.table(rid, 0):
                if p >= 0 and seen.setdefault(p, e["id"]) != e["id"]:
                    again += 1
                    seen[p] = e["id"]
        for rid in s["end"]:
            eng.release(rid)
    assert again > 0, "the trace was meant to hand pages of finished requests to later ones"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(workdir, dtype):
    """bin/trace_run as a child process: mixed trace, default page size, exactly --max-tokens of cache."""
    raw, page, folder, reqs, ref = cached_setup(workdir, "B", dtype)
    steps = replay.mixed(reqs)
    out = os.path.join(str(workdir), f"trace_{dtype}")
    got = replay.run_trace_tool(folder, dtype, steps, out, replay.tokens_needed(steps, 64), raw["vocab_size"])
    for rid in reqs:
        assert tiny.max_abs(got[rid], ref[rid]) < bound_of("B", dtype, rid), rid
    # a step in which nothing is wanted writes no file; a request may end in a step without entries
    steps2 = [{"step": 0, "entries": [{"id": "x", "tokens": reqs["r1"][:9], "want": []}], "end": []},
              {"step": 1, "entries": [{"id": "x", "tokens": reqs["r1"][9:], "want": [len(reqs["r1"]) - 10]}], "end": []},
              {"step": 2, "entries": [], "end": ["x"]}]
    out2 = os.path.join(str(workdir), f"trace2_{dtype}")
    got2 = replay.run_trace_tool(folder, dtype, steps2, out2, 64, raw["vocab_size"])
    assert not os.path.exists(os.path.join(out2, "0.f32"))
    assert tiny.max_abs(got2["x"][0], ref["r1"][-1]) < bound_of("B", dtype, "r1")


def test_out_of_pages_is_an_error_and_changes_nothing(workdir):
    from rust_mlx_b200.cache import OutOfPages
    raw, page, folder, reqs, ref = cached_setup(workdir, "A", "float32")
    eng = engine_for(folder, "float32", page, 32)           # two pages of 16
    eng.step([("a", reqs["r1"][:10], [])])
    with pytest.raises(OutOfPages):
        eng.step([("a", reqs["r1"][10:17], []), ("b", reqs["r2"][:20], [])])
    assert eng.length("a") == 10 and eng.length("b") == 0
    eng.pools.table.check()
    assert eng.pools.table.free_pages(0) == 1
    got = eng.step([("a", reqs["r1"][10:], [6])])
    assert tiny.max_abs(got[0].cpu(), ref["r1"][-1]) < TOL["float32"]
    with pytest.raises(ValueError, match="vocabulary"):
        eng.step([("a", [3], []), ("c", [raw["vocab_size"]], [0])])
    assert eng.length("c") == 0 and eng.length("a") == 17


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("D", "float32"), ("D", "bfloat16")])
def test_named_intermediates_of_a_step_match_the_plain_implementation(workdir, name, dtype):
    """``bin/trace_run --dump-intermediates``: every layer run's named tensors of a whole-prompt step against the
    plain implementation's tensors of the same names (what the reference's trace program does with an oracle's
    dump, src/bin/trace.rs:4-24), and of a later decoded token against the plain tensors' row of that position."""
    from safetensors.torch import load_file
    raw, page, folder, reqs, ref = cached_setup(workdir, name, dtype)
    toks = reqs["r4"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:-1], "want": [0]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[-1:], "want": [0]}], "end": ["a"]}]
    out = os.path.join(str(workdir), f"dump_{name}_{dtype}")
    replay.run_trace_tool(folder, dtype, steps, out, 64, raw["vocab_size"], extra=["--dump-intermediates", "all", "--page-size", str(page)])
    want = {}
    plain.PlainModel(folder, rounding=None if dtype == "float32" else "bfloat16").logits(toks, want)
    first = load_file(os.path.join(out, "0.intermediates.safetensors"))
    last = load_file(os.path.join(out, "1.intermediates.safetensors"))
    names = {f"run{i}.{n}" for i in range(raw["num_hidden_layers"])
             for n in ("residual", "norm1", "qkv", "q_rot", "attn_out", "mixer_out", "norm2", "ffn_act", "ffn_out")}
    assert set(first) == names
    # (a decoding step with heads of 128 in bfloat16 rotates inside its attention kernel: no q_rot then)
    assert set(last) | {n for n in names if n.endswith("q_rot")} == names
    tol = 2e-5 if dtype == "float32" else 4e-2
    for got, rows in ((first, slice(0, len(toks) - 1)), (last, slice(len(toks) - 1, len(toks)))):
        for key, t in got.items():
            w = want[key][rows].float()
            assert t.shape == w.shape, key
            assert tiny.max_abs(t, w) < tol * max(1.0, w.abs().max().item()), key


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_context_in_portions_and_then_token_by_token(workdir, dtype):
    """4,400 tokens on configuration D (heads of 128): the prompt in portions of 512 (each portion's attention sees
    thousands of earlier keys, so a tile's keys are shared among several blocks and their shares added), then 24
    tokens one by one (the decoding attention splits 70 key tiles among a cluster), beside a second, short request
    that decodes in the same steps.  Against the plain implementation evaluated once over the whole sequence in
    float64 on the GPU (sharpened weights, as everywhere in this file: a few keys carry most of a row's weight)."""
    raw, page = tiny.CONFIGS["D"]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=8, store="float32"))
    n, tail = 4400, 24
    long_ids = tiny.prompts(raw["vocab_size"], [n], seed=11)[0]
    short_ids = tiny.prompts(raw["vocab_size"], [40 + tail], seed=12)[0]
    config, tensors = plain.read_folder(folder)
    rounding = None if dtype == "float32" else "bfloat16"
    w = {k: v.to("cuda:0") for k, v in plain.prepare_weights(config, tensors, rounding).items()}
    exact = {k: v.to("cuda:0") for k, v in plain.prepare_weights(config, tensors, None).items()}
    want = plain.forward(config, w, long_ids, rounding).float().cpu()
    want_exact = plain.forward(config, exact, long_ids, None).float().cpu()
    want_short = plain.forward(config, w, short_ids, rounding).float().cpu()
    eng = engine_for(folder, dtype, page, -(-n // page) * page + 2 * page)
    got, got_short = [], []
    at = 0
    while at < n - tail:
        c = min(512, n - tail - at)
        rows = eng.step([("long", long_ids[at:at + c], [c - 1])])
        got.append((at + c - 1, rows[0].cpu()))
        at += c
    eng.step([("short", short_ids[:40], [])])
    for i in range(tail):
        rows = eng.step([("long", long_ids[at + i:at + i + 1], [0]), ("short", short_ids[40 + i:41 + i], [0])])
        got.append((at + i, rows[0].cpu()))
        got_short.append((40 + i, rows[1].cpu()))
    eng.release("long")
    eng.release("short")
    assert eng.pools.table.live() == 0
    tol = 1e-4 if dtype == "float32" else max(TOL[dtype], tiny.max_abs(want, want_exact))
    for pos, row in got:
        assert tiny.max_abs(row, want[pos]) < tol, (pos, tol)
    for pos, row in got_short:
        assert tiny.max_abs(row, want_short[pos]) < (1e-4 if dtype == "float32" else TOL[dtype]), pos


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("head_dim, heads, kv_heads, hidden", [(48, 5, 5, 72), (80, 6, 2, 104), (112, 7, 1, 88), (144, 3, 3, 120),
                                                               (256, 4, 2, 136)])
def test_head_sizes_in_steps_of_16_and_odd_head_counts(workdir, head_dim, heads, kv_heads, hidden, dtype):
    """Head sizes that no tensor-core attention kernel is built for (48, 80, 112, 144, 256), head counts and groups
    that are no power of two, widths that are multiples of 8 only: the engine takes them (the attention on FMA
    units where nothing faster exists) and agrees with the plain implementation, mixed and with the tail token by
    token; nothing is computed wrongly for lack of a kernel."""
    raw = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=2, hidden_size=hidden,
               num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=152,
               vocab_size=211, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=4096)
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=head_dim, store="float32"))
    reqs = {f"r{i}": p for i, p in enumerate(tiny.prompts(raw["vocab_size"], [37, 5, 70, 18], seed=head_dim))}
    pm = plain.PlainModel(folder, rounding=None if dtype == "float32" else "bfloat16")
    exact = plain.PlainModel(folder)
    for way in ("mixed", "tail_one_by_one"):
        steps = getattr(replay, way)(reqs)
        got = replay.run_engine(engine_for(folder, dtype, 16, replay.tokens_needed(steps, 16)), steps)
        for rid, toks in reqs.items():
            want = pm.logits(toks).float()
            tol = 2e-5 if dtype == "float32" else max(TOL[dtype], tiny.max_abs(want, exact.logits(toks).float()))
            assert tiny.max_abs(got[rid], want) < tol, (way, rid)
