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


class _Launched:
    """A step that is on its way: which requests want a token from it, and where the tokens will arrive."""

    __slots__ = ("wanting", "host", "event", "t0")

    def __init__(self, wanting, host, event, t0):
        self.wanting, self.host, self.event, self.t0 = wanting, host, event, t0


def generate(engine, prompts: list, *, max_tokens: int = 256, temperature: float = 0.0, seed: int = 0,
             ignore_eos: bool = False, prefill_chunk: int = 128, max_batch_tokens: int | None = None,
             max_seqs: int | None = None, max_context: int = 0, eos_token_ids=None,
             run_ahead: bool = True, on_token=None) -> GenerationResult:
    """Generate up to ``max_tokens`` tokens after each prompt (lists of token ids).

    An end-of-sequence token ends a request and is not part of its output, as in the
    reference (src/bin/infer.rs:172-176).  ``temperature`` may be one number or one per
    prompt; 0 is greedy.

    ``run_ahead``: the next step is launched before the host has read the tokens of the step
    before: a decoding request's next id is taken on the device from where the sampling left
    it, so the host's work for a step (scheduling, tables, launch) hides behind the GPU's work
    on the step before.  A request that turns out to have ended (end-of-sequence) has then
    been given one step too many; that step's token is dropped and its cache position is
    never read.

    ``on_token(i, token)`` is called for every token of prompt ``i`` as soon as the host has
    it (the reference's ``--stream`` prints pieces at that moment, src/bin/infer.rs:177-185)."""
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
    # the scheduler refuses at ``add`` what the engine could not hold later: the caller's limit or the engine's own
    # (its graphs' block tables are made for that many positions; the last generated token is never fed, so a
    # request may count one token more than the cache ever holds of it), whichever is smaller
    limit = min(x for x in (max_context, engine.max_context + 1) if x > 0)
    sched = Scheduler(engine.pools.table, max_seqs=max_seqs, max_batch_tokens=budget, prefill_chunk=prefill_chunk,
                      max_context=limit)
    rids = [engine._rid(("generate", id(sched), i)) for i in range(n)]
    index = {rid: i for i, rid in enumerate(rids)}
    known = [list(p) for p in prompts]      # token ids the host knows
    out = [[] for _ in range(n)]
    reasons = ["length"] * n
    done = [False] * n
    owed = [0] * n                          # tokens sampled on the device that the host has not read yet (0 or 1)
    res = GenerationResult(out, reasons, prompt_tokens=sum(len(p) for p in prompts))
    result_buf = torch.zeros(max_seqs + 1, dtype=torch.int32, device=engine.device)
    stream = torch.cuda.current_stream()
    first_done = 0
    t_first = None

    def launch(entries) -> _Launched:
        """Build the batch of ``entries`` and put it on the stream; the tokens travel to pinned memory behind it."""
        t0 = time.perf_counter()
        seqs, wanting = [], []
        # a portion that starts at position 0 belongs to a request that was just admitted (or admitted again after
        # it had stepped back): the scheduler gave it a slot, whose fixed-size state starts from zero
        engine.pools.reset_state([engine.pools.table.slot(e.req) for e in entries if e.start == 0])
        for e in entries:
            i = index[e.req]
            from_last = owed[i] > 0 and e.start + e.count > len(known[i])
            toks = [0] if from_last else known[i][e.start:e.start + e.count]
            seqs.append(SequenceInput(e.req, e.start, toks, [e.count - 1] if e.wants_logits else [], from_last))
            if e.wants_logits:
                wanting.append(i)
        t_list = [temps[i] for i in wanting]
        u_list = [uniform(seed, i, len(out[i]) + owed[i]) if temps[i] > 0 else 0.0 for i in wanting]
        if engine.graphs is not None and len(wanting) == len(entries) and all(e.count == 1 for e in entries):
            result = engine.graphs.run(seqs, t_list, u_list)              # a decode step: one captured graph
        else:
            batch = build_batch(seqs, engine.pools, engine.device, engine._status, engine.vocab_size, t_list, u_list)
            logits = engine.forward(batch)
            if wanting:
                engine.ops.sample(logits, batch.temperatures, batch.uniforms, result_buf[1:1 + len(wanting)],
                                  batch.row_slots, engine.last_tokens)
            result_buf[0:1].copy_(engine._status)
            result = result_buf
        host = torch.empty(1 + len(wanting), dtype=torch.int32, pin_memory=True)
        host.copy_(result[:1 + len(wanting)], non_blocking=True)
        event = torch.cuda.Event()
        event.record(stream)
        return _Launched(wanting, host, event, t0)

    def harvest(step: _Launched) -> None:
        """Wait for a step's tokens and hand them to their requests."""
        nonlocal first_done, t_first
        step.event.synchronize()                                          # the step's one synchronisation
        host = step.host.tolist()
        if host[0] != 0:
            engine.check_status()
        for i, tok in zip(step.wanting, host[1:]):
            ahead = owed[i] > 0
            owed[i] = 0
            if done[i]:
                continue                                                  # a step too many for a request that had ended
            if tok in eos:
                reasons[i] = "stop"
                done[i] = True
                sched.finish(rids[i])
                continue
            if not out[i]:
                first_done += 1
            out[i].append(tok)
            known[i].append(tok)
            if on_token is not None:
                on_token(i, tok)
            if len(out[i]) >= max_tokens:
                done[i] = True
                sched.finish(rids[i])
            elif not ahead:
                sched.append_token(rids[i])
        res.steps += 1
        now = time.perf_counter()
        res.step_seconds.append(now - step.t0)
        if t_first is None and all(out[i] or done[i] for i in range(n)):
            t_first = now

    try:
        for i, p in enumerate(prompts):
            sched.add(rids[i], len(p), max_tokens)
        t_start = time.perf_counter()
        pending = None
        while pending is not None or not sched.idle():
            if pending is None:
                entries = sched.next()
                res.preemptions += len(sched.take_preempted())
                if not entries:
                    raise RuntimeError("the scheduler has requests but could build no step")
                pending = launch(entries)
                sched.step_done()
            # the step after `pending`, launched before its tokens are read where that is possible: requests that
            # will get a token from `pending` and need more are counted as having it
            following = None
            if run_ahead:
                hopeful = [i for i in pending.wanting if not done[i] and len(out[i]) + 1 < max_tokens]
                for i in hopeful:
                    sched.append_token(rids[i])
                    owed[i] = 1
                entries = sched.next() if hopeful or not sched.idle() else []
                preempted = sched.take_preempted()
                res.preemptions += len(preempted)
                if entries and not preempted:
                    following = launch(entries)
                    sched.step_done()
                    harvest(pending)
                else:
                    # a request that was put back needs its tokens on the host to be computed again: read them first
                    harvest(pending)
                    if entries:
                        alive = [e for e in entries if not done[index[e.req]]]
                        if alive:
                            following = launch(alive)
                        sched.step_done()
            else:
                harvest(pending)
            pending = following
        t_end = time.perf_counter()
        res.prefill_seconds = (t_first or t_end) - t_start
        res.decode_seconds = t_end - (t_first or t_end)
        res.generated_tokens = sum(len(o) for o in out)
        return res
    finally:
        torch.cuda.synchronize()
        for rid in rids:
            if engine.pools.table.has(rid):
                engine.pools.table.close(rid)
        for i in range(n):
            engine._req_ids.pop(("generate", id(sched), i), None)
