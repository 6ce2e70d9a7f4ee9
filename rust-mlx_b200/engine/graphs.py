"""Decode steps as CUDA graphs.

A decode step (every sequence brings one token and wants its logits) launches a
few hundred small kernels; issuing them one by one costs more host time than
the GPU needs to run them.  The step — embedding, every layer, final norm, head
and sampling — is captured once per (batch size, what the parts say of their launch shapes: ``Part.graph_key``) into a
CUDA graph whose kernels read the step's ids, positions, block tables and
sampling numbers from one device buffer of fixed address and layout; each later
step of that shape copies its numbers into the buffer and launches the graph.
Graphs are dropped when a workspace buffer they point into is reallocated.
"""
from __future__ import annotations

import gc

import torch

from ..parts.base import DecodeShape, Part
from .batch import BatchLayout, check_sequences


# Batch sizes that graphs exist for: a step of n sequences runs in the next size up, the spare
# places repeating the first sequence (the same token to the same position, sampled with the same
# numbers: the same values are written twice and the spare results are ignored).  At most half as many places again.
_BUCKETS = [1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512]


def bucket(n: int) -> int:
    for b in _BUCKETS:
        if n <= b:
            return b
    return n


class _Captured:
    __slots__ = ("graph", "layout", "hosts", "events", "turn", "dev", "result", "generation", "batch")


class DecodeGraphs:
    def __init__(self, engine, max_graphs: int = 32):
        self.engine = engine
        self.max_graphs = max_graphs
        self.graphs = {}
        self.replays = 0
        self.captures = 0
        # the parts whose launches follow the sequences' lengths: they say so by overriding ``graph_key``
        self._keyed = [p for p in engine.spec.all_parts() if type(p).graph_key is not Part.graph_key]

    def entries(self) -> list:
        e = self.engine
        return [max(1, -(-e.max_context // e.pools.page_size)) for _ in e.pools.paged_groups]

    def run(self, seqs: list, temperatures, uniforms) -> torch.Tensor:
        """One decode step of ``seqs`` (one token each).  Returns the device tensor
        [status, token_0, ...] (it may be longer than the batch: spare places follow the
        real ones); the caller copies it to the host."""
        e = self.engine
        check_sequences(seqs)
        n_real = len(seqs)
        spare = min(bucket(len(seqs)), e.pools.max_requests + len(seqs)) - len(seqs)
        if spare > 0:
            seqs = list(seqs) + [seqs[0]] * spare
            # a spare place samples with the first sequence's own numbers and leaves its choice in the scrap word
            # after the last state slot, never in the first sequence's word of ``last_tokens``
            temperatures = list(temperatures) + [temperatures[0]] * spare if temperatures is not None else None
            uniforms = list(uniforms) + [uniforms[0]] * spare if uniforms is not None else None
        n = len(seqs)
        longest = max(s.start + 1 for s in seqs)
        if longest > e.max_context:
            raise ValueError(f"a sequence of {longest} tokens exceeds the context limit {e.max_context}")
        shape = DecodeShape(n, longest)
        key = (n, tuple(p.graph_key(shape) for p in self._keyed))
        cap = self.graphs.get(key)
        if cap is not None and cap.generation != e.workspace.generation:
            del self.graphs[key]
            cap = None
        if cap is None:
            cap = self._capture(seqs, temperatures, uniforms, key, n_real)
        # staging buffers take turns, so that a caller who does not wait for each step's result
        # never overwrites numbers whose copy to the device is still to come
        cap.turn = (cap.turn + 1) % len(cap.hosts)
        host, event = cap.hosts[cap.turn], cap.events[cap.turn]
        event.synchronize()
        facts = cap.layout.fill(host.numpy(), seqs, e.pools, e.vocab_size, temperatures, uniforms)
        cap.layout.part(host.numpy(), 10)[n_real:] = e.pools.max_requests
        cap.batch.max_seq_len = facts["max_seq_len"]
        cap.dev.copy_(host, non_blocking=True)
        event.record()
        cap.graph.replay()
        self.replays += 1
        e.ops.count_launches(e._launches_per_graph.get(key, 0))
        return cap.result

    def _capture(self, seqs, temperatures, uniforms, key, n_real=None) -> _Captured:
        e = self.engine
        n = len(seqs)
        if len(self.graphs) >= self.max_graphs:
            self.graphs.pop(next(iter(self.graphs)))
        cap = _Captured()
        cap.layout = BatchLayout(n, n, n, self.entries())
        cap.hosts = [torch.empty(cap.layout.total, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        cap.events = [torch.cuda.Event() for _ in cap.hosts]
        cap.turn = 0
        cap.dev = torch.zeros(cap.layout.total, dtype=torch.int32, device=e.device)
        cap.result = torch.zeros(n + 1, dtype=torch.int32, device=e.device)
        facts = cap.layout.fill(cap.hosts[0].numpy(), seqs, e.pools, e.vocab_size, temperatures, uniforms)
        cap.layout.part(cap.hosts[0].numpy(), 10)[n if n_real is None else n_real:] = e.pools.max_requests
        cap.dev.copy_(cap.hosts[0], non_blocking=True)
        cap.events[0].record()
        cap.batch = cap.layout.views(cap.dev, e._status, facts)
        # once eagerly: buffers reach their size, kernels' attributes are set, libraries warm up.
        # It writes this step's keys and values, which the replay below writes again, the same; the tokens it
        # chooses are put back, because a step that runs ahead takes its ids from there.
        saved = e.last_tokens.clone()
        self._step(cap)
        e.last_tokens.copy_(saved)
        torch.cuda.synchronize()
        cap.generation = e.workspace.generation
        e.workspace.frozen = True
        # While a stream is being captured nothing may free pinned memory, events or graphs: the collector
        # could do just that in the middle of the capture if it found an engine that is no longer used (its
        # staging buffers and graphs) and so make the capture invalid.  It runs now and rests meanwhile.
        collecting = gc.isenabled()
        gc.collect()
        gc.disable()
        try:
            before = e.ops.launch_count
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._step(cap)
            e._launches_per_graph[key] = e.ops.launch_count - before
        finally:
            if collecting:
                gc.enable()
            e.workspace.frozen = False
        cap.graph = graph
        self.graphs[key] = cap
        self.captures += 1
        return cap

    def _step(self, cap) -> None:
        e = self.engine
        logits = e.forward(cap.batch)
        e.ops.sample(logits, cap.batch.temperatures, cap.batch.uniforms, cap.result[1:], cap.batch.row_slots, e.last_tokens)
        cap.result[0:1].copy_(e._status)
