"""Generation: the scheduler above the step function.

The loop of the reference's command line is prefill in chunks, then argmax and a
one-token forward per token (src/bin/infer.rs:155-191), for one request.  Here
the scheduler builds each step's batch from all live requests (decoded tokens
first, then portions of prompts under the token budget), the step function runs
it, the sampler picks a token for every request whose last known token was in
the batch, and one copy brings the tokens (and the kernels' status word) to the
host.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch

from ..sampling.rng import uniform
from .batch import SequenceInput, build_batch
from .scheduler import Scheduler


@dataclass
class GenerationResult:
    tokens: list                      # per request: generated token ids
    finish_reasons: list              # per request: "stop" (end-of-sequence token) or "length"
    prompt_tokens: int = 0
    generated_tokens: int = 0
    steps: int = 0
    prefill_seconds: float = 0.0      # until every request has its first token
    decode_seconds: float = 0.0       # the rest
    step_seconds: list = field(default_factory=list)
    preemptions: int = 0


def generate(engine, prompts: list, *, max_tokens: int = 256, temperature: float = 0.0, seed: int = 0,
             ignore_eos: bool = False, prefill_chunk: int = 128, max_batch_tokens: int | None = None,
             max_seqs: int | None = None, max_context: int = 0, eos_token_ids=None) -> GenerationResult:
    """Generate up to ``max_tokens`` tokens after each prompt (lists of token ids).

    An end-of-sequence token ends a request and is not part of its output, as in the
    reference (src/bin/infer.rs:172-176).  ``temperature`` may be one number or one per
    prompt; 0 is greedy."""
    if max_tokens <= 0 or prefill_chunk <= 0:
        raise ValueError("max_tokens and prefill_chunk must be positive")
    n = len(prompts)
    temps = list(temperature) if isinstance(temperature, (list, tuple)) else [float(temperature)] * n
    if len(temps) != n:
        raise ValueError("one temperature per prompt, or one for all")
    eos = set(engine.spec.eos_token_ids if eos_token_ids is None else eos_token_ids)
    if ignore_eos:
        eos = set()
    for p in prompts:
        if any((not isinstance(t, int)) or t < 0 or t >= engine.vocab_size for t in p):
            raise ValueError("token outside vocabulary")
    max_seqs = max_seqs or min(engine.pools.max_requests, max(n, 1))
    budget = max_batch_tokens or max(prefill_chunk, max_seqs)
    sched = Scheduler(engine.pools.table, max_seqs=max_seqs, max_batch_tokens=budget, prefill_chunk=prefill_chunk,
                      max_context=max_context)
    rids = [engine._rid(("generate", id(sched), i)) for i in range(n)]
    index = {rid: i for i, rid in enumerate(rids)}
    known = [list(p) for p in prompts]
    out = [[] for _ in range(n)]
    reasons = ["length"] * n
    try:
        for i, p in enumerate(prompts):
            sched.add(rids[i], len(p), max_tokens)
        res = GenerationResult(out, reasons, prompt_tokens=sum(len(p) for p in prompts))
        result_buf = torch.zeros(max_seqs + 1, dtype=torch.int32, device=engine.device)
        first_done = 0
        t_start = time.perf_counter()
        t_first = None
        while not sched.idle():
            t0 = time.perf_counter()
            entries = sched.next()
            res.preemptions += len(sched.take_preempted())
            if not entries:
                raise RuntimeError("the scheduler has requests but could build no step")
            seqs, wanting = [], []
            for e in entries:
                i = index[e.req]
                seqs.append(SequenceInput(e.req, e.start, known[i][e.start:e.start + e.count],
                                          [e.count - 1] if e.wants_logits else []))
                if e.wants_logits:
                    wanting.append(i)
            t_list = [temps[i] for i in wanting]
            u_list = [uniform(seed, i, len(out[i])) if temps[i] > 0 else 0.0 for i in wanting]
            if engine.graphs is not None and len(wanting) == len(entries) and all(e.count == 1 for e in entries):
                result = engine.graphs.run(seqs, t_list, u_list)          # a decode step: one captured graph
                host = result.tolist()                                    # the step's one synchronisation
            else:
                batch = build_batch(seqs, engine.pools, engine.device, engine._status, engine.vocab_size, t_list, u_list)
                logits = engine.forward(batch)
                if wanting:
                    engine.ops.sample(logits, batch.temperatures, batch.uniforms, result_buf[1:1 + len(wanting)])
                result_buf[0:1].copy_(engine._status)
                host = result_buf[:1 + len(wanting)].tolist()             # the step's one synchronisation
            if host[0] != 0:
                engine.check_status()
            sched.step_done()
            for i, tok in zip(wanting, host[1:]):
                if tok in eos:
                    reasons[i] = "stop"
                    sched.finish(rids[i])
                    continue
                if not out[i]:
                    first_done += 1
                out[i].append(tok)
                known[i].append(tok)
                if len(out[i]) >= max_tokens:
                    sched.finish(rids[i])
                else:
                    sched.append_token(rids[i])
            res.steps += 1
            now = time.perf_counter()
            res.step_seconds.append(now - t0)
            if t_first is None and (first_done == n or sched.idle() or all(out[i] or reasons[i] == "stop" for i in range(n))):
                t_first = now
        t_end = time.perf_counter()
        res.prefill_seconds = (t_first or t_end) - t_start
        res.decode_seconds = t_end - (t_first or t_end)
        res.generated_tokens = sum(len(o) for o in out)
        return res
    finally:
        for rid in rids:
            if engine.pools.table.has(rid):
                engine.pools.table.close(rid)
        for i in range(n):
            engine._req_ids.pop(("generate", id(sched), i), None)
