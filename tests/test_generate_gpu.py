"""Generation through the entry points against the plain implementation."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as plain
import tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def workdir(tmp_path_factory):
    return tmp_path_factory.mktemp("generate")


def engine(folder, dtype, page, tokens=2048, requests=8):
    from rust_mlx_b200.engine import Engine
    return Engine(folder, dtype=dtype, max_tokens=tokens, page_size=page, max_requests=requests)


@pytest.mark.parametrize("name, lengths, n, chunk", [("A", [5, 17, 33], 8, 7), ("B", [1, 9, 24, 40], 6, 5)])
def test_greedy_generation_equals_the_plain_implementation(workdir, name, lengths, n, chunk):
    raw, page = tiny.CONFIGS[name]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=11))
    ps = tiny.prompts(raw["vocab_size"], lengths, seed=5)
    pm = plain.PlainModel(folder)
    want = [pm.greedy(p, n) for p in ps]
    eng = engine(folder, "float32", page)
    assert eng.generate(ps, max_tokens=n, prefill_chunk=chunk) == want                  # one mixed batch
    assert [eng.generate([p], max_tokens=n, prefill_chunk=1000)[0] for p in ps] == want  # each alone, whole
    assert eng.generate(ps, max_tokens=n, prefill_chunk=1, max_batch_tokens=3) == want   # token by token
    eng.pools.table.check()
    assert eng.pools.table.live() == 0


def test_bfloat16_greedy_follows_the_plain_bfloat16_restatement(workdir):
    raw, page = tiny.CONFIGS["A"]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=11))
    ps = tiny.prompts(raw["vocab_size"], [5, 17, 33], seed=5)
    pm = plain.PlainModel(folder, rounding="bfloat16")
    eng = engine(folder, "bfloat16", page)
    got = eng.generate(ps, max_tokens=8, prefill_chunk=7)
    for p, g in zip(ps, got):
        ids = list(p)
        for t in g:   # every chosen token must be (nearly) the plain argmax given the same history
            logits = pm.logits(ids)[-1]
            assert logits[t] >= logits.max() - 2e-2
            ids.append(t)


@pytest.mark.parametrize("name", ["C", "D", "E"])
def test_bfloat16_generation_at_real_head_sizes(workdir, name):
    """Heads of 64 and of 128 in bfloat16 through ``generate``: decode steps are captured graphs (batch sizes
    that change as requests end), the decoding attention splits the keys of the longer requests and, with heads
    of 128, norms and rotates its own token; every chosen token must be (nearly) the plain argmax given the
    same history, and generation in lockstep without graphs must choose the same tokens."""
    raw, page = tiny.CONFIGS[name]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=21))
    ps = tiny.prompts(raw["vocab_size"], [300, 5, 129, 64, 230], seed=9)
    pm = plain.PlainModel(folder, rounding="bfloat16")
    eng = engine(folder, "bfloat16", page, tokens=4096)
    limits = [24, 9, 17, 30, 12]
    # a short request first: its decode graph points into a workspace that the longer prompts then outgrow
    first = eng.generate([ps[1]], max_tokens=4, ignore_eos=True)[0]
    r = eng.generate(ps, max_tokens=max(limits), prefill_chunk=96, ignore_eos=True)
    assert r[1][:4] == first
    for i, (p, g) in enumerate(zip(ps, r)):
        ids = list(p)
        for t in g[:limits[i]]:
            logits = pm.logits(ids)[-1]
            assert logits[t] >= logits.max() - 4e-2, (name, i, len(ids))
            ids.append(t)
    graphs, eng.graphs = eng.graphs, None
    assert eng.generate(ps, max_tokens=max(limits), prefill_chunk=96, ignore_eos=True, run_ahead=False) == r
    eng.graphs = graphs


def test_graph_capture_is_not_disturbed_by_the_collector(workdir):
    """Garbage that holds pinned memory and events (what an engine that is no longer used leaves behind) and a
    collector set to run at every opportunity: freeing such things while a decode step is being captured would
    make the capture invalid, so the capture collects first and keeps the collector off meanwhile."""
    import gc
    raw, page = tiny.CONFIGS["D"]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=21))
    ps = tiny.prompts(raw["vocab_size"], [40, 70, 9], seed=2)
    eng = engine(folder, "bfloat16", page, tokens=1024)

    class Holder:
        pass
    for _ in range(64):
        h = Holder()
        h.me, h.buf, h.event = h, torch.empty(4096, dtype=torch.int32, pin_memory=True), torch.cuda.Event()
    del h
    old = gc.get_threshold()
    gc.set_threshold(1, 1, 1)
    try:
        got = eng.generate(ps, max_tokens=6, ignore_eos=True)
    finally:
        gc.set_threshold(*old)
    assert eng.graphs is not None and eng.graphs.captures > 0
    graphs, eng.graphs = eng.graphs, None
    assert eng.generate(ps, max_tokens=6, ignore_eos=True, run_ahead=False) == got
    eng.graphs = graphs


def test_long_decoding_and_the_first_tokens(workdir):
    """200 decoded tokens across many page edges, teacher-forced against the plain logits, and
    the very first positions of a sequence (one token, two tokens)."""
    raw, page = tiny.CONFIGS["B"]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=4))
    ids = tiny.prompts(raw["vocab_size"], [260], seed=9)[0]
    ref = plain.PlainModel(folder).logits(ids).float()
    eng = engine(folder, "float32", page, tokens=264)
    first = eng.step([("s", ids[:1], [0])]).cpu()
    assert tiny.max_abs(first[0], ref[0]) < 2e-5
    second = eng.step([("s", ids[1:2], [0])]).cpu()
    assert tiny.max_abs(second[0], ref[1]) < 2e-5
    eng.step([("s", ids[2:60], [])])
    for i in range(60, 260):
        row = eng.step([("s", ids[i:i + 1], [0])]).cpu()
        assert tiny.max_abs(row[0], ref[i]) < 2e-5, i
    eng.release("s")
    two = eng.step([("t", ids[:2], [0, 1])]).cpu()
    assert tiny.max_abs(two, ref[:2]) < 2e-5


def test_long_greedy_generation_with_a_window(workdir):
    raw, page = tiny.CONFIGS["Bw"]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=12))
    p = tiny.prompts(raw["vocab_size"], [30], seed=2)[0]
    want = plain.PlainModel(folder).greedy(p, 60)
    eng = engine(folder, "float32", page, tokens=96)
    assert eng.generate([p], max_tokens=60, prefill_chunk=16)[0] == want


def test_running_ahead_changes_nothing_but_the_time(workdir):
    """With run_ahead the next step is launched before the host reads the last step's tokens (ids are taken on the
    device); the tokens must be the same, also when requests end at different times, stop at an end-of-sequence
    token, sample with a temperature, or are put back for lack of pages."""
    raw, page = tiny.CONFIGS["D"]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=13))
    ps = tiny.prompts(raw["vocab_size"], [30, 7, 65, 18], seed=4)
    for dtype in ("float32", "bfloat16"):
        eng = engine(folder, dtype, page, tokens=1024)
        for opts in (dict(max_tokens=12), dict(max_tokens=9, temperature=0.8, seed=5), dict(max_tokens=20, prefill_chunk=16)):
            a = eng.generate_detailed(ps, run_ahead=True, **opts)
            b = eng.generate_detailed(ps, run_ahead=False, **opts)
            assert a.tokens == b.tokens and a.finish_reasons == b.finish_reasons
        base = eng.generate(ps, max_tokens=12, run_ahead=False)
        stop = base[2][5]
        a = eng.generate_detailed(ps, max_tokens=12, eos_token_ids=[stop], run_ahead=True)
        b = eng.generate_detailed(ps, max_tokens=12, eos_token_ids=[stop], run_ahead=False)
        assert a.tokens == b.tokens and a.finish_reasons == b.finish_reasons and "stop" in a.finish_reasons
        assert eng.pools.table.live() == 0
    small = engine(folder, "float32", page, tokens=256)        # four pages of 64: requests are put back
    ps2 = tiny.prompts(raw["vocab_size"], [60, 58, 50], seed=6)
    a = small.generate_detailed(ps2, max_tokens=40, prefill_chunk=32, run_ahead=True)
    b = small.generate_detailed(ps2, max_tokens=40, prefill_chunk=32, run_ahead=False)
    assert a.tokens == b.tokens and a.preemptions > 0 and b.preemptions > 0
    assert small.pools.table.live() == 0 and small.pools.table.free_pages(0) == 4


def test_eos_stops_and_is_not_part_of_the_output(workdir):
    raw, page = tiny.CONFIGS["A"]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=11))
    p = tiny.prompts(raw["vocab_size"], [17], seed=5)[0]
    pm = plain.PlainModel(folder)
    want = pm.greedy(p, 8)
    eng = engine(folder, "float32", page)
    stop_at = want[3]
    cut = want.index(stop_at)
    r = eng.generate_detailed([p], max_tokens=8, eos_token_ids=[stop_at])
    assert r.tokens[0] == want[:cut] and r.finish_reasons == ["stop"]
    r = eng.generate_detailed([p], max_tokens=8, eos_token_ids=[stop_at], ignore_eos=True)
    assert r.tokens[0] == want and r.finish_reasons == ["length"]


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(workdir):
    raw, page = tiny.CONFIGS["B"]
    folder = tiny.make_folder(workdir, raw, seed=11)
    ps = tiny.prompts(raw["vocab_size"], [1, 9, 24, 40], seed=5)
    eng = engine(folder, "float32", page)
    a = eng.generate(ps, max_tokens=6, temperature=0.7, seed=3, prefill_chunk=5)
    b = eng.generate(ps, max_tokens=6, temperature=0.7, seed=3, prefill_chunk=40)
    c = eng.generate(ps, max_tokens=6, temperature=0.7, seed=4, prefill_chunk=5)
    assert a == b and a != c
    # request 0 alone draws the same numbers as request 0 in the batch
    assert eng.generate(ps[:1], max_tokens=6, temperature=0.7, seed=3)[0] == a[0]
    # every drawn token is the inverse-CDF choice of the plain softmax with the same uniform
    from rust_mlx_b200.sampling import uniform
    pm = plain.PlainModel(folder)
    ids = list(ps[1])
    for step, t in enumerate(a[1]):
        p = torch.softmax(pm.logits(ids)[-1] / 0.7, -1)
        cdf = torch.cumsum(p, 0)
        u = uniform(3, 1, step)
        lo = cdf[t - 1].item() if t > 0 else 0.0
        assert lo - 1e-4 <= u <= cdf[t].item() + 1e-4
        ids.append(t)
    mixed = eng.generate(ps, max_tokens=6, temperature=[0.0, 0.7, 0.0, 0.7], seed=3)
    greedy = eng.generate(ps, max_tokens=6)
    assert mixed[0] == greedy[0] and mixed[2] == greedy[2] and mixed[1] == a[1]


@pytest.mark.parametrize("n_prompts", [5, 7])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_at_batch_sizes_between_graph_sizes(workdir, n_prompts, dtype):
    """Five and seven requests decode in graphs made for six and eight: the spare places repeat the first request.
    A spare place must not leave a token of its own where the first request's next step looks for its id, so
    running a step ahead, in lockstep, with and without graphs all draw the same tokens; in float32 every drawn
    token is the inverse-CDF choice of the plain softmax for the same uniform number."""
    from rust_mlx_b200.sampling import uniform
    raw, page = tiny.CONFIGS["D"]
    folder = tiny.make_folder(workdir, raw, seed=17)
    ps = tiny.prompts(raw["vocab_size"], [9, 30, 3, 17, 65, 12, 40][:n_prompts], seed=3)
    eng = engine(folder, dtype, page, tokens=2048)
    opts = dict(max_tokens=14, temperature=0.8, seed=9, ignore_eos=True)
    a = eng.generate(ps, run_ahead=True, **opts)
    assert eng.graphs is not None and eng.graphs.replays > 0
    assert any(k[0] == n_prompts + 1 for k in eng.graphs.graphs)   # the padded size was used
    b = eng.generate(ps, run_ahead=False, **opts)
    graphs, eng.graphs = eng.graphs, None
    c = eng.generate(ps, run_ahead=True, **opts)
    d = eng.generate(ps, run_ahead=False, **opts)
    eng.graphs = graphs
    assert a == b == c == d
    assert len({tuple(t) for t in a}) > 1 and a != eng.generate(ps, **dict(opts, temperature=0.0))
    if dtype == "float32":
        pm = plain.PlainModel(folder)
        for i in (0, 1, n_prompts - 1):
            ids = list(ps[i])
            for step, t in enumerate(a[i]):
                cdf = torch.cumsum(torch.softmax(pm.logits(ids)[-1] / 0.8, -1), 0)
                u = uniform(9, i, step)
                lo = cdf[t - 1].item() if t > 0 else 0.0
                assert lo - 1e-4 <= u <= cdf[t].item() + 1e-4, (i, step)
                ids.append(t)


@pytest.mark.parametrize("name", ["C", "D"])
def test_forty_requests_decode_together(workdir, name):
    """Forty live requests: decode graphs of 48 places and fewer as requests end, products of 17 to 64 rows
    (the tcgen05 product's wider tiles or the library's product), decoding attention that does not split its
    keys.  float32: the plain implementation's greedy tokens; bfloat16, with graphs and in lockstep without:
    every chosen token is (nearly) the argmax of the plain bfloat16 restatement given the same history."""
    import random
    rng = random.Random(5)
    raw, page = tiny.CONFIGS[name]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=23))
    lengths = [rng.choice([3, 9, 17, 33, 64, 65, 100]) for _ in range(40)]
    ps = tiny.prompts(raw["vocab_size"], lengths, seed=6)
    limits = [rng.randint(4, 12) for _ in range(40)]
    pm = plain.PlainModel(folder)
    want = [pm.greedy(p, n) for p, n in zip(ps, limits)]
    eng = engine(folder, "float32", page, tokens=40 * 128, requests=48)
    got = eng.generate(ps, max_tokens=12, prefill_chunk=256, max_batch_tokens=512, ignore_eos=True)
    assert [g[:n] for g, n in zip(got, limits)] == want
    assert max(k[0] for k in eng.graphs.graphs) >= 40
    eng16 = engine(folder, "bfloat16", page, tokens=40 * 128, requests=48)
    got16 = eng16.generate(ps, max_tokens=12, prefill_chunk=256, max_batch_tokens=512, ignore_eos=True)
    assert max(k[0] for k in eng16.graphs.graphs) >= 40
    graphs, eng16.graphs = eng16.graphs, None
    plain16 = eng16.generate(ps, max_tokens=12, prefill_chunk=256, max_batch_tokens=512, ignore_eos=True, run_ahead=False)
    eng16.graphs = graphs
    pm16 = plain.PlainModel(folder, rounding="bfloat16")
    for i in range(0, 40, 3):
        for out in (got16, plain16):
            ids = list(ps[i])
            for t in out[i][:limits[i]]:
                logits = pm16.logits(ids)[-1]
                assert logits[t] >= logits.max() - 4e-2, (name, i, len(ids))
                ids.append(t)


def test_a_request_beyond_the_engines_context_is_refused_at_once(workdir):
    """``generate`` hands the engine's own context limit to the scheduler: a request that would outgrow it is
    refused before anything runs, not in the middle of generation."""
    from rust_mlx_b200.engine import Engine
    from rust_mlx_b200.engine.scheduler import RequestRejected
    raw, page = tiny.CONFIGS["A"]
    folder = tiny.make_folder(workdir, raw, seed=11)
    eng = Engine(folder, dtype="float32", max_tokens=1024, page_size=page, max_requests=4, max_context=40)
    ps = tiny.prompts(raw["vocab_size"], [10, 30], seed=1)
    with pytest.raises(RequestRejected):
        eng.generate(ps, max_tokens=12)          # 30 + 12 > 40 + 1
    assert eng.pools.table.live() == 0
    assert len(eng.generate(ps, max_tokens=11, ignore_eos=True)[1]) == 11


def test_pages_run_out_during_generation_requests_are_computed_again(workdir):
    raw, page = tiny.CONFIGS["A"]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=11))
    ps = tiny.prompts(raw["vocab_size"], [30, 28, 25], seed=8)
    pm = plain.PlainModel(folder)
    want = [pm.greedy(p, 24) for p in ps]
    eng = engine(folder, "float32", page, tokens=112)        # 7 pages of 16: not enough for all three to finish together
    r = eng.generate_detailed(ps, max_tokens=24, prefill_chunk=16)
    assert r.tokens == want
    assert r.preemptions > 0
    assert eng.pools.table.live() == 0 and eng.pools.table.free_pages(0) == 7


@pytest.mark.parametrize("name, seed", [("A", 1), ("A", 2), ("B", 3), ("Bw", 4), ("C", 5), ("E", 6)])
def test_random_workloads_through_the_scheduler(workdir, name, seed):
    """A dozen requests of random lengths through ``generate`` with random portions, budgets and seats, in a
    cache too small for all of them (so that requests wait, are preempted and computed again), running a step
    ahead and in lockstep: in float32 every request's greedy tokens are the plain implementation's."""
    import random
    rng = random.Random(seed)
    raw, page = tiny.CONFIGS[name]
    folder = tiny.sharpen(tiny.make_folder(workdir, raw, seed=40 + seed))
    lengths = [rng.choice([1, 2, 3, 7, 16, 17, 31, 40, 64, 65, 90]) for _ in range(12)]
    ps = tiny.prompts(raw["vocab_size"], lengths, seed=seed)
    n = rng.randint(3, 20)
    pm = plain.PlainModel(folder)
    want = [pm.greedy(p, n) for p in ps]
    longest = -(-(max(lengths) + n) // page) * page
    for run_ahead in (True, False):
        tokens = longest + rng.randint(1, 6) * page                 # room for the longest request and a little more
        eng = engine(folder, "float32", page, tokens=tokens, requests=rng.randint(2, 6))
        chunk = rng.choice([1, 3, 8, 32, 200])
        r = eng.generate_detailed(ps, max_tokens=n, prefill_chunk=chunk, max_batch_tokens=rng.choice([None, chunk + 4]),
                                  run_ahead=run_ahead)
        assert r.tokens == want, (run_ahead, tokens, chunk)
        eng.pools.table.check()
        assert eng.pools.table.live() == 0 and eng.pools.table.free_pages(0) == eng.pools.num_pages


def test_python_entry_point_and_command_line(workdir):
    import rust_mlx_b200
    raw, page = tiny.CONFIGS["A"]
    folder = tiny.make_folder(workdir, raw, seed=11)
    p = tiny.prompts(raw["vocab_size"], [12], seed=5)[0]
    want = plain.PlainModel(folder).greedy(p, 5)
    assert rust_mlx_b200.generate(folder, [p], dtype="float32", max_tokens=5, page_size=page) == [want]
    ids = os.path.join(str(workdir), "prompt.json")
    json.dump(p, open(ids, "w"))
    out = os.path.join(str(workdir), "report.json")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "infer"), "--model", folder, "--prompt-ids", ids, "--max-tokens", "5",
           "--runs", "2", "--warmup-tokens", "2", "--prefill-chunk", "4", "--ignore-eos", "--dtype", "float32",
           "--page-size", str(page), "--output", out]
    subprocess.run(cmd, check=True, timeout=300)
    report = json.load(open(out))
    assert [r["tokens"] for r in report["runs"]] == [want, want]
    assert report["prompt_ids"] == p and report["runs"][0]["generated_tokens"] == 5
    env = report["environment"]          # hardware, software, revision (with its dirty flag), what the GPU was doing
    assert "B200" in env["hardware"]["gpu"] and env["software"]["torch"] and "dirty" in env["revision"]
    assert "sm_mhz" in env["workload"] or env["workload"].get("clocks") == "unavailable"
    assert report["runtime"]["tuning"]["policy"] == "auto"
    assert subprocess.run(cmd[:-2] + ["--runs", "0"], capture_output=True).returncode != 0
    # --stream: the timed runs' ids on standard output as they come, and no report there
    streamed = subprocess.run(cmd[:-2] + ["--stream"], capture_output=True, text=True, timeout=300, check=True).stdout
    assert [[int(t) for t in line.split()] for line in streamed.strip().splitlines()] == [want, want]


def test_refusals(workdir):
    from rust_mlx_b200.engine import Engine, EngineError
    from rust_mlx_b200.engine.scheduler import RequestRejected
    raw, page = tiny.CONFIGS["A"]
    folder = tiny.make_folder(workdir, raw, seed=11)
    with pytest.raises(EngineError):
        Engine(folder, dtype="float16")
    with pytest.raises(EngineError):
        Engine(folder, page_size=24)
    eng = engine(folder, "float32", page, tokens=32)
    with pytest.raises(RequestRejected):
        eng.generate([list(range(40))], max_tokens=4)
    with pytest.raises(RequestRejected):
        eng.generate([[]], max_tokens=4)
    with pytest.raises(ValueError):
        eng.generate([[1, 2, 999]], max_tokens=4)
    assert eng.pools.table.live() == 0
