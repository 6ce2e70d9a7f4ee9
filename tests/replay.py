"""Ways of cutting the same requests into steps, and running them through the engine.

A step is {"step": i, "entries": [{"id", "tokens", "want"}], "end": [...]}, the format
bin/trace_run reads.  Every token's logits are wanted, so that the result of each way is
one [length, vocab] tensor per request.
"""
import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def whole(requests: dict) -> list:
    """Each request alone and whole, one after the other."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def tail_one_by_one(requests: dict, tail: int = 32) -> list:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        cuts = [head] + [1] * (len(toks) - head)
        steps += _alone(rid, toks, cuts, len(steps))
    return steps


def portions(requests: dict, sizes=(7, 2, 13, 3, 2, 5, 1, 11)) -> list:
    """Portions of changing size, down to two tokens and one."""
    steps = []
    for k, (rid, toks) in enumerate(requests.items()):
        cuts, left, i = [], len(toks), k
        while left > 0:
            c = min(left, sizes[i % len(sizes)])
            cuts.append(c)
            left -= c
            i += 1
        steps += _alone(rid, toks, cuts, len(steps))
    return steps


def _alone(rid, toks, cuts, first_step):
    steps, at = [], 0
    for j, c in enumerate(cuts):
        last = at + c == len(toks)
        steps.append({"step": first_step + j, "entries": [{"id": rid, "tokens": toks[at:at + c],
                                                           "want": list(range(c))}], "end": [rid] if last else []})
        at += c
    return steps


def mixed(requests: dict, live: int = 4, sizes=(5, 1, 9, 2, 1, 1, 6, 3, 1, 1, 1, 4)) -> list:
    """Up to ``live`` requests at a time; every step gives each live request a portion whose
    size walks through ``sizes`` (ones are decoded tokens beside portions of the others);
    a request that ends makes room for the next, which then takes over its pages."""
    waiting = list(requests.items())
    running = []  # [rid, toks, at, size index]
    steps = []
    k = 0
    while waiting or running:
        while waiting and len(running) < live:
            rid, toks = waiting.pop(0)
            running.append([rid, toks, 0, k])
            k += 3
        entries, end = [], []
        skipping = [(len(steps) + r[3]) % 5 == 4 for r in running]
        for r, skip in zip(running, skipping):
            rid, toks, at, si = r
            if skip and not all(skipping):
                continue  # a request may be left out of a step and go on later
            c = min(len(toks) - at, sizes[(len(steps) + si) % len(sizes)])
            entries.append({"id": rid, "tokens": toks[at:at + c], "want": list(range(c))})
            r[2] = at + c
            if r[2] == len(toks):
                end.append(rid)
        running = [r for r in running if r[2] < len(r[1])]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def random_cuts(requests: dict, seed: int, live: int = 4, largest: int = 300) -> list:
    """Up to ``live`` requests at a time, every step a random choice of them (at least one), each with a
    portion of random size: mostly single tokens and small portions, now and then one of up to ``largest``."""
    rng = np.random.RandomState(seed)
    waiting = list(requests.items())
    running = []  # [rid, toks, at]
    steps = []
    while waiting or running:
        while waiting and len(running) < live:
            rid, toks = waiting.pop(0)
            running.append([rid, toks, 0])
        chosen = [r for r in running if rng.rand() < 0.7] or [running[rng.randint(len(running))]]
        entries, end = [], []
        for r in chosen:
            kind = rng.rand()
            c = 1 if kind < 0.4 else int(rng.randint(2, 20)) if kind < 0.75 else int(rng.randint(20, largest + 1))
            c = min(c, len(r[1]) - r[2])
            entries.append({"id": r[0], "tokens": r[1][r[2]:r[2] + c], "want": list(range(c))})
            r[2] += c
            if r[2] == len(r[1]):
                end.append(r[0])
        running = [r for r in running if r[2] < len(r[1])]
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def tokens_needed(steps: list, page: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``page``."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // page) * page for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def run_engine(engine, steps: list) -> dict:
    """Drive ``engine.step``; returns request -> [length, vocab] float32 logits (CPU)."""
    rows = {}
    for s in steps:
        entries = [(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        logits = engine.step(entries, s["end"]).cpu()
        at = 0
        for e in s["entries"]:
            n = len(e["want"])
            rows.setdefault(e["id"], []).append(logits[at:at + n])
            at += n
    return {rid: torch.cat(parts) for rid, parts in rows.items()}


def run_trace_tool(folder: str, dtype: str, steps: list, out_dir: str, max_tokens: int, vocab: int,
                   extra=()) -> dict:
    """Drive bin/trace_run as a child process, one step at a time, waiting for "done"."""
    cmd = [os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens), *extra]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    rows = {}
    try:
        for s in steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"trace_run said {line!r}"
            n = sum(len(e["want"]) for e in s["entries"])
            if n:
                data = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(n, vocab)
                at = 0
                for e in s["entries"]:
                    k = len(e["want"])
                    rows.setdefault(e["id"], []).append(torch.from_numpy(data[at:at + k].copy()))
                    at += k
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    return {rid: torch.cat(parts) for rid, parts in rows.items()}
