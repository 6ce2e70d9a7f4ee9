"""The ``infer`` command line, after the reference's (src/bin/infer.rs:14-56).

Kept from the reference, with its names, defaults and meanings: ``--model`` (the
folder), ``--prompt-ids`` (a JSON file holding an array of token ids),
``--max-tokens`` 256, ``--runs`` 3, ``--warmup-tokens`` 16, ``--prefill-chunk``
128, ``--ignore-eos``, ``--output`` (the JSON report; standard output if absent).
runs, max-tokens and prefill-chunk must be positive (src/bin/infer.rs:62-65); one
warm-up run of ``--warmup-tokens`` tokens comes before the timed runs (108-112,
150-154) and every run starts from an empty cache (155).  ``--stream`` prints the
tokens of the timed runs as they are generated (the reference prints their text,
177-185: here token ids, space separated, ``i:id`` when there are several prompts)
and, like the reference, leaves the report out of standard output (222).  Text
prompts and chat templates need a tokenizer and are not offered: prompts are
token ids.  Added: ``--dtype``, ``--temperature``, ``--seed``, ``--random-weights``,
``--page-size``, ``--cache-tokens``, ``--max-batch-tokens``, ``--tuning``; ``--prompt-ids`` may
also hold an array of arrays, which are then generated as one batch.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="infer", description="generate tokens with the B200 engine")
    ap.add_argument("--model", required=True, help="folder with config.json and safetensors")
    ap.add_argument("--prompt-ids", required=True, help="JSON file: an array of token ids (or an array of such arrays)")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--runs", type=int, default=3)
    ap.add_argument("--warmup-tokens", type=int, default=16)
    ap.add_argument("--prefill-chunk", type=int, default=128)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--output", help="write the JSON report here instead of standard output")
    ap.add_argument("--stream", action="store_true", help="print token ids as they are generated (timed runs only)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--temperature", type=float, default=0.0, help="0 is greedy")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--random-weights", action="store_true", help="read config.json only and draw weights from --seed")
    ap.add_argument("--page-size", type=int, default=64)
    ap.add_argument("--cache-tokens", type=int, default=0, help="tokens the cache holds (default: what the prompts need)")
    ap.add_argument("--max-batch-tokens", type=int, default=0, help="token budget of a step (default: the prefill chunk)")
    ap.add_argument("--tuning", default="auto",
                    help="which products of few rows take the tcgen05 kernel: auto (timed at start), measured (a fixed "
                         "rule), all, none, or the JSON report of an earlier run whose choices are made again")
    return ap


def main(argv=None) -> int:
    a = build_parser().parse_args(argv)
    if a.runs <= 0 or a.max_tokens <= 0 or a.prefill_chunk <= 0:
        print("error: runs/tokens/chunk must be positive", file=sys.stderr)
        return 2
    with open(a.prompt_ids) as fh:
        ids = json.load(fh)
    if not isinstance(ids, list) or not ids:
        print("error: empty prompt", file=sys.stderr)
        return 2
    prompts = ids if isinstance(ids[0], list) else [ids]
    if any(not p for p in prompts):
        print("error: empty prompt", file=sys.stderr)
        return 2

    import torch
    from ..engine import Engine

    page = a.page_size
    need = sum(-(-(len(p) + a.max_tokens) // page) * page for p in prompts)
    t0 = time.time()
    tuning = a.tuning
    if tuning not in ("auto", "measured", "all", "none"):
        with open(tuning) as fh:
            tuning = json.load(fh)["runtime"]["tuning"]
    engine = Engine(a.model, dtype=a.dtype, random_weights=a.random_weights, seed=a.seed, page_size=page,
                    max_tokens=a.cache_tokens or need, max_requests=max(len(prompts), 1), verbose=True, tuning=tuning)
    load_seconds = time.time() - t0
    print(f"weights ready: {load_seconds:.3f}s, {torch.cuda.memory_allocated() / 2**30:.2f} GiB active",
          file=sys.stderr)
    options = dict(temperature=a.temperature, seed=a.seed, ignore_eos=a.ignore_eos, prefill_chunk=a.prefill_chunk,
                   max_batch_tokens=a.max_batch_tokens or None)
    records = []
    for run in range(a.runs + 1):
        warmup = run == 0
        limit = a.warmup_tokens if warmup else a.max_tokens
        torch.cuda.reset_peak_memory_stats()
        on_token = None
        if a.stream and not warmup:
            def on_token(i, tok):
                print(f"{i}:{tok}" if len(prompts) > 1 else tok, end=" ", flush=True)
        r = engine.generate_detailed(prompts, max_tokens=max(limit, 1), on_token=on_token, **options)
        if on_token is not None:
            print(flush=True)
        tps = (r.generated_tokens - len(prompts)) / r.decode_seconds if r.decode_seconds > 0 else 0.0
        print(f"{'warmup' if warmup else 'run'} {run}: prompt={r.prompt_tokens} output={r.generated_tokens} "
              f"prefill={r.prefill_seconds:.3f}s decode={tps:.2f} tok/s", file=sys.stderr)
        if not warmup:
            records.append({
                "run": run, "prompt_tokens": r.prompt_tokens, "generated_tokens": r.generated_tokens,
                "tokens": r.tokens if len(prompts) > 1 else r.tokens[0], "finish_reasons": r.finish_reasons,
                "prefill_seconds": r.prefill_seconds, "decode_seconds": r.decode_seconds,
                "prefill_tokens_per_second": r.prompt_tokens / r.prefill_seconds if r.prefill_seconds > 0 else None,
                "decode_tokens_per_second": tps, "inter_token_seconds": r.step_seconds, "steps": r.steps,
                "preemptions": r.preemptions, "peak_memory_bytes": torch.cuda.max_memory_allocated()})
    from .environment import capture
    report = {
        "environment": capture(),
        "model": a.model,
        "runtime": {"backend": "cuda sm_100a", "dtype": a.dtype, "temperature": a.temperature, "seed": a.seed,
                    "batch_size": len(prompts), "kv_cache": "fresh per run", "ignore_eos": a.ignore_eos,
                    "prefill_chunk": a.prefill_chunk, "warmup_tokens": a.warmup_tokens, "page_size": page,
                    "random_weights": a.random_weights,
                    # which products took which kernel: pass this table as ``tuning`` to get the same bits again
                    "tuning": engine.tuning_table()},
        "prompt_ids": ids, "load_seconds": load_seconds, "runs": records}
    text = json.dumps(report, indent=1)
    if a.output:
        with open(a.output, "w") as fh:
            fh.write(text)
    elif not a.stream:
        print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
