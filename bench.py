"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]

The default run has the layer sizes of Qwen3-8B with random weights in bfloat16: decode at
batch 8 from a context of 2,048 tokens per request.  It prints ONE JSON line.  ``value`` is
decoded tokens per second, timed on the device with CUDA events over exactly K steps (each
step: upload of the step's ids and tables from pinned memory, the model, greedy sampling).
``e2e`` is the same through the Python entry point (``Engine.generate``): host token ids in,
host token ids out, one host synchronisation per step; the ids it generated are then compared
with those of its warm-up run and of a run without graphs and in lockstep (``checked``), as
the reference's benchmarks compare every timed run's ids with the first run's
(src/bin/batch-bench.rs:147-151).  ``prefill`` is one 2,048-token prompt in one step;
``roofline`` is the decode step's bytes (every weight once plus the live requests' cache)
over its time.  Weights (15 GB) are far larger than L2, so no flush is needed between steps.

``--per-kernel`` instead times the phases of one decode step one by one (CUDA events between
the kernels, inside a captured graph, so without host gaps and without overlap between
neighbouring kernels) and prints bytes, time and fraction of the memory peak of each: a
synchronised diagnostic, not shares of the natural run time (the reference's
src/bin/profile.rs:22-36 does the same per phase).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
                vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                max_position_embeddings=4096)
# the Qwen3-4B and Qwen3-32B layer sizes beside the default
SHAPES = {
    "qwen3-8b": QWEN3_8B,
    "qwen3-4b": dict(QWEN3_8B, hidden_size=2560, intermediate_size=9728, tie_word_embeddings=True),
    "qwen3-32b": dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600),
}
CONTEXT = 2048          # tokens each request holds when decoding starts
MAX_CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = 64


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(path):
        try:
            raw = json.load(open(path))
            out["hbm_gbs"] = float(raw.get("hbm_gbs", out["hbm_gbs"]))
            out["bf16_tflops"] = float(raw.get("bf16_tflops_sustained", raw.get("bf16_tflops", out["bf16_tflops"])))
            out["source"] = "measured"
        except Exception:
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def model_bytes(cfg, layers):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qkv = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"] * h
    o = cfg["num_attention_heads"] * cfg["head_dim"] * h
    per_layer = qkv + o + 3 * h * i
    params = layers * per_layer + v * h           # the head once; embedding rows are a few KB
    return params * 2, per_layer, v * h


def kv_bytes_per_token(cfg, layers):
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, layers, tokens):
    _, per_layer, head = model_bytes(cfg, layers)
    gemm = 2.0 * tokens * layers * per_layer + 2.0 * head          # logits for the last row only
    attn = 2.0 * tokens * tokens * cfg["head_dim"] * cfg["num_attention_heads"] * layers   # causal: half of 4 T^2 d
    return gemm + attn


class DecodeRun:
    """B live requests holding CONTEXT tokens each (synthetic cache), stepped one token at a time."""

    def __init__(self, engine, batch, context):
        import torch
        self.e, self.batch, self.context, self.torch = engine, batch, context, torch
        self.rids = list(range(10_000, 10_000 + batch))
        self.len = context
        for r in self.rids:
            engine.pools.open(r)
            engine.pools.table.reserve(r, context)
            engine.pools.table.commit(r, context)
        g = torch.Generator().manual_seed(batch)
        self.ids = torch.randint(0, engine.vocab_size, (4096, batch), generator=g).tolist()
        self.out = torch.empty(batch, dtype=torch.int32, device=engine.device)
        self.n = 0

    def step(self):
        from rust_mlx_b200.engine.batch import SequenceInput, build_batch
        e = self.e
        for r in self.rids:
            e.pools.table.reserve(r, self.len + 1)
        toks = self.ids[self.n % len(self.ids)]
        seqs = [SequenceInput(r, self.len, [toks[i]], [0]) for i, r in enumerate(self.rids)]
        if e.graphs is not None:      # what generation does for a decode step: one captured graph
            e.graphs.run(seqs, None, None)
        else:
            batch = build_batch(seqs, e.pools, e.device, e._status, e.vocab_size)
            logits = e.forward(batch)
            e.ops.sample(logits, None, None, self.out)
        self.len += 1
        self.n += 1
        for r in self.rids:
            e.pools.table.commit(r, self.len)

    def close(self):
        for r in self.rids:
            self.e.pools.table.close(r)


def time_decode(engine, batch, steps, warmup, clocks=None):
    import torch
    from rust_mlx_b200.kernels import ops
    run = DecodeRun(engine, batch, CONTEXT)
    try:
        for _ in range(warmup):
            run.step()
        torch.cuda.synchronize()
        if clocks:
            clocks.start()
        launches0 = ops.launch_count
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            run.step()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        engine.check_status()
        return ms, ops.launch_count - launches0, (clocks.stop() if clocks else None)
    finally:
        run.close()


def time_prefill(engine, tokens, reps=3, start_at=0):
    """One portion of ``tokens`` prompt tokens in one step, the request holding ``start_at`` tokens already (0: a whole
    prompt from its start; otherwise a later portion of a long prompt, its earlier keys being the synthetic cache)."""
    import torch
    from rust_mlx_b200.engine.batch import SequenceInput, build_batch
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, engine.vocab_size, (tokens,), generator=g).tolist()
    best = None
    for rep in range(reps + 1):
        rid = 20_000 + rep
        engine.pools.open(rid)
        if start_at:
            engine.pools.table.reserve(rid, start_at)
            engine.pools.table.commit(rid, start_at)
        engine.pools.table.reserve(rid, start_at + tokens)
        batch = build_batch([SequenceInput(rid, start_at, ids, [tokens - 1])], engine.pools, engine.device, engine._status,
                            engine.vocab_size)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.forward(batch)
        stop.record()
        torch.cuda.synchronize()
        engine.pools.table.close(rid)
        ms = start.elapsed_time(stop)
        if rep > 0:                      # the first repetition warms up
            best = ms if best is None else min(best, ms)
    engine.check_status()
    return best


def time_e2e(engine, batch, new_tokens):
    """Through the Python entry point: prompts of CONTEXT host token ids, ``new_tokens`` generated each."""
    import torch
    g = torch.Generator().manual_seed(7)
    prompts = torch.randint(0, engine.vocab_size, (batch, CONTEXT), generator=g).tolist()
    opts = dict(ignore_eos=True, prefill_chunk=2048, max_batch_tokens=batch * CONTEXT)
    # warm-up with the same shapes: the decode step of this batch size is captured into its graph here
    warm = engine.generate(prompts, max_tokens=3, **opts)
    r = engine.generate_detailed(prompts, max_tokens=new_tokens, **opts)
    decoded = r.generated_tokens - batch
    # what was generated: the timed run's ids begin with the warm-up run's, and a run of plain launches in
    # lockstep (no graphs, no step launched ahead) generates the same ids
    graphs, engine.graphs = engine.graphs, None
    try:
        plain = engine.generate(prompts, max_tokens=new_tokens, run_ahead=False, **opts)
    finally:
        engine.graphs = graphs
    checked = all(len(t) == new_tokens for t in r.tokens) and all(t[:3] == w for t, w in zip(r.tokens, warm)) and plain == r.tokens
    if not checked:
        first = next(((i, j) for i, (x, y) in enumerate(zip(r.tokens, plain)) for j, (u, v) in enumerate(zip(x, y)) if u != v), None)
        print(f"bench.py: the timed run's ids differ from the check runs' (first difference at request, token {first})",
              file=sys.stderr)
    # bytes per decode step: ids, positions, sequence indices, starts, lengths, slots, rows, block tables up; tokens + status down
    # a captured decode step uploads one buffer of fixed layout: ids, positions, sequence indices, starts, lengths,
    # slots, rows, temperatures, uniforms and block tables of the context limit
    from rust_mlx_b200.engine.batch import BatchLayout
    from rust_mlx_b200.engine.graphs import bucket
    b = bucket(batch)
    h2d = 4 * BatchLayout(b, b, b, [engine.max_context // PAGE for _ in engine.pools.paged_groups]).total
    d2h = 4 * (b + 1)
    return decoded / r.decode_seconds, h2d, d2h, checked


def per_kernel(engine, raw, a, pk):
    """One decode step of ``a.batch`` requests at CONTEXT tokens, captured with an event after every phase of every
    layer; replayed ``a.steps`` times.  Prints a table (standard error) and one JSON line."""
    import torch
    from rust_mlx_b200.engine.batch import SequenceInput, build_batch
    run = DecodeRun(engine, a.batch, CONTEXT)
    try:
        e = engine
        for r in run.rids:
            e.pools.table.reserve(r, run.len + 1)
        seqs = [SequenceInput(r, run.len, [run.ids[0][i]], [0]) for i, r in enumerate(run.rids)]
        batch = build_batch(seqs, e.pools, e.device, e._status, e.vocab_size)
        out = torch.empty(a.batch, dtype=torch.int32, device=e.device)
        marks = []          # (phase that ended here, event)

        def tap(name, tensor):
            ev = torch.cuda.Event(enable_timing=True, external=True)
            ev.record()
            marks.append((name, ev))

        def step():
            marks.clear()
            tap("start", None)
            tap("nothing", None)          # two events with no kernel between them: what an event itself costs
            logits = e.forward(batch)
            e.ops.sample(logits, None, None, out)
            tap("head", None)
        e.forward(batch)                      # buffers reach their size
        torch.cuda.synchronize()
        e._ctx.tap = tap
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
        finally:
            e._ctx.tap = None
        # what ends at a mark, by the mark's name: the kernels between it and the mark before
        phase = {"residual": None, "norm1": "add + norm", "qkv": "q/k/v product", "q_rot": "norm + rotation + cache write",
                 "attn_out": "attention", "mixer_out": "output product", "norm2": "add + norm", "ffn_act": "gate/up product + SwiGLU",
                 "ffn_out": "down product", "head": "final norm + head + sampling", "nothing": "(an event alone)"}
        total = {}
        for _ in range(max(a.warmup, 3)):
            graph.replay()
        for _ in range(a.steps):
            graph.replay()
            torch.cuda.synchronize()
            last = marks[0][1]
            for name, ev in marks[1:]:
                if phase.get(name) is None:
                    continue            # (the stream before a block's norm: the same place as its norm1 mark)
                total.setdefault(phase[name], []).append(last.elapsed_time(ev) * 1e3)
                last = ev
        h, inter, v = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
        nq, nkv, hd, layers = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"], a.layers
        per_layer_bytes = {"q/k/v product": (nq + 2 * nkv) * hd * h * 2, "output product": nq * hd * h * 2,
                           "gate/up product + SwiGLU": 2 * inter * h * 2, "down product": inter * h * 2,
                           "attention": a.batch * (CONTEXT + 1) * 2 * nkv * hd * 2,
                           "add + norm": a.batch * h * (4 + 4 + 2 + 2), "norm + rotation + cache write": a.batch * (nq + 2 * nkv) * hd * 4,
                           "final norm + head + sampling": v * h * 2 + a.batch * v * 8}
        rows, step_us = [], 0.0
        event_us = sum(total.pop("(an event alone)")) / a.steps      # subtracted from every phase below
        for name, times in total.items():
            calls = len(times) // a.steps
            us = max(sum(times) / a.steps / calls - event_us, 0.01)
            gbs = per_layer_bytes[name] / us / 1e3
            step_us += us * calls
            rows.append({"phase": name, "calls_per_step": calls, "us": round(us, 2), "bytes": per_layer_bytes[name],
                         "gb_per_s": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 3)})
        print(f"{'phase':34s} {'calls':>5s} {'us each':>9s} {'MB each':>9s} {'GB/s':>8s} {'of peak':>8s}", file=sys.stderr)
        for r_ in rows:
            print(f"{r_['phase']:34s} {r_['calls_per_step']:5d} {r_['us']:9.2f} {r_['bytes'] / 1e6:9.2f} {r_['gb_per_s']:8.1f} {r_['frac']:8.3f}",
                  file=sys.stderr)
        print(f"(an event alone: {event_us:.2f} us, subtracted from every phase)", file=sys.stderr)
        print(json.dumps({"per_kernel": rows, "step_us_serialised": round(step_us, 1), "event_us": round(event_us, 2), "batch": a.batch, "context": CONTEXT,
                          "layers": layers, "shape": a.shape, "peak_gb_per_s": pk["hbm_gbs"], "of": pk["source"],
                          "note": "events between kernels inside one captured graph: no host gaps, no overlap of neighbours"}))
        return 0
    finally:
        run.close()


def continuous(cfg, raw, a):
    """64 requests, prompts of 128..3072 uniform-random ids, 256 generated tokens each, through the scheduler:
    portions of prompts (at most 512 tokens a step) run beside the decoded tokens of the requests already past theirs."""
    import random

    import torch
    from rust_mlx_b200.engine import Engine
    rng = random.Random(0)
    lengths = [rng.randrange(128, 3073) for _ in range(64)]
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, raw["vocab_size"], (n,), generator=g).tolist() for n in lengths]
    new_tokens = 256
    cache_tokens = sum(-(-(n + new_tokens) // PAGE) * PAGE for n in lengths)
    engine = Engine(cfg, dtype="bfloat16", random_weights=True, seed=0, max_tokens=cache_tokens, page_size=PAGE, max_requests=64,
                    tuning=a.policy)
    opts = dict(max_tokens=new_tokens, ignore_eos=True, prefill_chunk=512, max_batch_tokens=512 + 64, max_seqs=64)
    engine.generate(prompts[:8], **dict(opts, max_tokens=8))            # warm-up: kernels, graphs of the first sizes
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    r = engine.generate_detailed(prompts, **opts)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    line = {"metric": "continuous batching: generated tok/s over the whole run", "value": round(r.generated_tokens / wall, 1),
            "unit": "tok/s", "impl": "ours", "n_gpus": 1, "dtype": "bf16", "data": "synthetic",
            "config": {"model": a.shape + " shape, random weights", "layers": a.layers, "requests": 64, "prompt_tokens": r.prompt_tokens,
                       "generated_tokens": r.generated_tokens, "prefill_chunk": 512, "max_batch_tokens": 576, "page_size": PAGE},
            "seconds": round(wall, 3), "steps": r.steps, "preemptions": r.preemptions,
            "total_tok_per_s": round((r.generated_tokens + r.prompt_tokens) / wall, 1)}
    print(json.dumps(line))
    return 0


def main():
    global CONTEXT, MAX_CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"])
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64, prefill and e2e")
    ap.add_argument("--prefill-only", action="store_true", help="time the 2,048-token prefill only (for profiling it)")
    ap.add_argument("--portion-at", type=int, default=0, metavar="CONTEXT",
                    help="instead: time one 512-token portion of a prompt whose first CONTEXT tokens are in the cache (chunked "
                         "prefill of a long prompt); prints its own JSON line")
    ap.add_argument("--per-kernel", action="store_true",
                    help="instead: time the phases of one decode step one by one and print each one's bytes, time and "
                         "fraction of the memory peak")
    ap.add_argument("--shape", default="qwen3-8b", choices=sorted(SHAPES), help="layer sizes (default: the Qwen3-8B shape)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="tokens each request holds when decoding starts")
    ap.add_argument("--continuous", action="store_true",
                    help="instead: 64 requests with prompts of 128..3072 random ids, 256 tokens each, through the "
                         "scheduler with chunked prefill of 512 (continuous batching); prints its own JSON line")
    ap.add_argument("--policy", default="auto", choices=["auto", "measured", "all", "none"],
                    help="which products of few rows take the tcgen05 kernel (auto: time both when the engine starts)")
    a = ap.parse_args()
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust/MLX/Metal program for Apple GPUs: no Rust toolchain, no MLX and no "
                          "setup.py/pyproject.toml here (pip: 'not installable'), so it cannot be built or run on this box"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    a.warmup = max(a.warmup, 3)

    import torch
    from rust_mlx_b200.config import Qwen3Config
    from rust_mlx_b200.engine import Engine

    CONTEXT = a.context
    base = SHAPES[a.shape]
    if a.shape != "qwen3-8b" and a.layers == QWEN3_8B["num_hidden_layers"]:
        a.layers = base["num_hidden_layers"]
    MAX_CONTEXT = max(MAX_CONTEXT, 2 * CONTEXT)
    raw = dict(base, num_hidden_layers=a.layers, max_position_embeddings=MAX_CONTEXT)
    cfg = Qwen3Config.from_dict(raw)
    if a.continuous:
        return continuous(cfg, raw, a)
    if a.portion_at:
        CONTEXT = a.portion_at
    biggest = 1 if (a.no_points or a.prefill_only or a.per_kernel or a.portion_at) else max(64, a.batch)
    cache_tokens = max(biggest, a.batch) * (CONTEXT + 2 * PAGE + a.steps + a.warmup + 64)
    engine = Engine(cfg, dtype="bfloat16", random_weights=True, seed=0, max_tokens=cache_tokens, page_size=PAGE,
                    max_requests=max(biggest, a.batch) + 2, tuning=a.policy)
    for grp in engine.pools.paged_groups:      # synthetic cache contents for the requests that start at CONTEXT
        grp.k_pool.normal_(0, 1)
        grp.v_pool.normal_(0, 1)
    pk = peaks()
    if a.per_kernel:
        return per_kernel(engine, raw, a, pk)
    if a.portion_at:
        portion = 512
        ms = time_prefill(engine, portion, start_at=a.portion_at)
        _, per_layer, head = model_bytes(raw, a.layers)
        gemm = 2.0 * portion * a.layers * per_layer + 2.0 * head
        # every query of the portion against the cache's keys and, causally, the portion's own (half of them on average)
        attn = 4.0 * portion * (a.portion_at + portion / 2) * raw["head_dim"] * raw["num_attention_heads"] * a.layers
        print(json.dumps({"metric": f"prompt portion of {portion} tokens at context {a.portion_at} ({a.shape} shape, bf16)",
                          "value": round(portion / (ms * 1e-3), 1), "unit": "tok/s", "ms": round(ms, 3), "layers": a.layers,
                          "tflop": round((gemm + attn) / 1e12, 2), "attention_share_of_flop": round(attn / (gemm + attn), 3),
                          "frac": round((gemm + attn) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "of": pk["source"]}))
        return 0
    if a.prefill_only:
        pf_ms = time_prefill(engine, PREFILL_TOKENS)
        flops = prefill_flops(raw, a.layers, PREFILL_TOKENS)
        print(json.dumps({"prefill": {"value": round(PREFILL_TOKENS / (pf_ms * 1e-3), 1), "tokens": PREFILL_TOKENS,
                                      "ms": round(pf_ms, 3), "layers": a.layers,
                                      "frac": round(flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}}))
        return 0

    clocks = ClockSampler()
    ms, launches, clock_info = time_decode(engine, a.batch, a.steps, a.warmup, clocks)
    value = a.batch * 1000.0 / ms
    weight_bytes, _, _ = model_bytes(raw, a.layers)
    step_bytes = weight_bytes + a.batch * (CONTEXT + a.warmup + a.steps / 2) * kv_bytes_per_token(raw, a.layers)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {a.batch}, context {CONTEXT} ({a.shape} shape, bf16)", "value": round(value, 2), "unit": "tok/s",
        "n_gpus": 1, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": a.shape + " shape, random weights", "layers": a.layers, "layers_full": base["num_hidden_layers"],
                   "hidden": raw["hidden_size"], "q_heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"],
                   "head_dim": raw["head_dim"], "intermediate": raw["intermediate_size"],
                   "vocab": raw["vocab_size"], "global_batch": a.batch, "seq_len": CONTEXT, "max_context": MAX_CONTEXT,
                   "page_size": PAGE, "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 ({weight_bytes / 1e9:.0f} GB of weights per step), no flush",
                   "peaks": pk["source"]},
        "gpu_launches": launches, "clocks": clock_info,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]},
    }
    if not a.no_points:
        points = {}
        for b in (1, 64):
            pms, _, _ = time_decode(engine, b, max(8, a.steps // 2), a.warmup)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 2)
        line["points"] = points
        pf_ms = time_prefill(engine, PREFILL_TOKENS)
        flops = prefill_flops(raw, a.layers, PREFILL_TOKENS)
        line["prefill"] = {"value": round(PREFILL_TOKENS / (pf_ms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3),
                           "frac": round(flops / (pf_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4), "of": pk["source"]}
        e2e, h2d, d2h, checked = time_e2e(engine, a.batch, max(128, a.steps))
        line["e2e"] = {"value": round(e2e, 2), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
        line["checked"] = checked
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
