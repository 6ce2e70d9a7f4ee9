"""One step's batch: a flat list of tokens from several requests and what kernels
need to know about them, uploaded to the device in a single copy.

Per token: its id, its absolute position and the index of its sequence in the
batch.  Per sequence: where its tokens start in the flat list (``q_start``), its
length after this step (``seq_lens``), its state slot, and per paged cache group
its block table.  ``logit_rows`` are the flat indices of the tokens whose logits
are wanted.  Two float rows (temperatures and uniform numbers for sampling) ride
in the same buffer.  The reference runs either one request's tokens or several
requests' single tokens at one offset (src/dense.rs:371, src/batching.rs:34-53);
here any mix is one batch.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class SequenceInput:
    """One request's part of a step: ``tokens`` go to positions start .. start + len - 1."""

    req: int
    start: int
    tokens: list
    want: list = field(default_factory=list)  # indices into ``tokens`` whose logits are wanted
    from_last: bool = False  # the (single) token's id is what the last step's sampling left on the device


@dataclass
class StepBatch:
    n_tokens: int
    n_seqs: int
    n_rows: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    seq_index: torch.Tensor
    q_start: torch.Tensor
    seq_lens: torch.Tensor
    slots: torch.Tensor
    logit_rows: torch.Tensor
    block_tables: list
    status: torch.Tensor
    temperatures: torch.Tensor
    uniforms: torch.Tensor
    from_last: torch.Tensor     # int32 [tokens]: 1 where the id comes from the last step's sampling, on the device
    row_slots: torch.Tensor     # int32 [rows]: the state slot of the sequence of every wanted row
    any_from_last: bool
    q_start_host: list
    seq_lens_host: list
    start_host: list
    slots_host: list
    max_q_len: int
    max_seq_len: int
    # what parts form once per step and share between layers (the rotation's cosines and sines); emptied by the
    # engine at the start of every forward pass
    per_step: dict = field(default_factory=dict)
    # int32 [state slots] on the device: the token the last sampling chose for the request in each slot (the engine's)
    last_tokens: torch.Tensor = None

    @property
    def all_decode(self) -> bool:
        return self.max_q_len == 1


class BatchLayout:
    """Where each array lies in the one int32 buffer of a batch of given sizes."""

    def __init__(self, n_tokens: int, n_seqs: int, n_rows: int, entries: list):
        self.n_tokens, self.n_seqs, self.n_rows, self.entries = n_tokens, n_seqs, n_rows, list(entries)
        rows = max(n_rows, 1)
        self.sizes = [n_tokens, n_tokens, n_tokens, n_seqs + 1, n_seqs, n_seqs, rows, rows, rows, n_tokens, rows] + \
                     [n_seqs * e for e in entries]
        self.first_table = 11
        # every array starts on a 16-byte boundary
        self.offsets, at = [], 0
        for n in self.sizes:
            self.offsets.append(at)
            at += -(-n // 4) * 4
        self.total = at

    def part(self, buf, i, n=None):
        return buf[self.offsets[i]:self.offsets[i] + (self.sizes[i] if n is None else n)]

    def fill(self, buf: np.ndarray, seqs: list, pools, vocab_size: int, temperatures=None, uniforms=None) -> dict:
        """Write the arrays of ``seqs`` into ``buf`` (int32, ``total`` long); returns host-side facts."""
        counts = [len(s.tokens) for s in seqs]
        if self.n_tokens == self.n_seqs == self.n_rows and max(counts) == 1 and all(s.want == [0] for s in seqs):
            return self._fill_decode(buf, seqs, pools, vocab_size, temperatures, uniforms)
        q_start, rows = [0], []
        for s, c in zip(seqs, counts):
            for w in s.want:
                if not 0 <= w < c:
                    raise ValueError(f"request {s.req!r} wants logits at place {w} of {c} tokens")
                rows.append(q_start[-1] + w)
            q_start.append(q_start[-1] + c)
        ids = np.fromiter((t for s in seqs for t in s.tokens), dtype=np.int64, count=self.n_tokens)
        if ids.min() < 0 or ids.max() >= vocab_size:
            raise ValueError("token outside vocabulary")
        self.part(buf, 0)[:] = ids
        pos, sidx = self.part(buf, 1), self.part(buf, 2)
        for i, (s, c) in enumerate(zip(seqs, counts)):
            pos[q_start[i]:q_start[i + 1]] = np.arange(s.start, s.start + c, dtype=np.int32)
            sidx[q_start[i]:q_start[i + 1]] = i
        self.part(buf, 3)[:] = q_start
        seq_lens = [s.start + c for s, c in zip(seqs, counts)]
        self.part(buf, 4)[:] = seq_lens
        table = pools.table
        slots = [table.slot(s.req) for s in seqs]
        self.part(buf, 5)[:] = slots
        self.part(buf, 6)[:len(rows)] = rows
        fl = self.part(buf, 7).view(np.float32)
        fl[:] = 0.0
        if temperatures is not None:
            fl[:len(temperatures)] = temperatures
        fl = self.part(buf, 8).view(np.float32)
        fl[:] = 0.0
        if uniforms is not None:
            fl[:len(uniforms)] = uniforms
        fromlast = self.part(buf, 9)
        fromlast[:] = 0
        row_slots = []
        for i, (s, c) in enumerate(zip(seqs, counts)):
            if s.from_last:
                if c != 1:
                    raise ValueError("only a single decoded token can take its id from the last step")
                fromlast[q_start[i]] = 1
            row_slots += [slots[i]] * len(s.want)
        self.part(buf, 10)[:len(row_slots)] = row_slots
        for g, grp in enumerate(pools.paged_groups):
            e = self.entries[g]
            tab = self.part(buf, self.first_table + g).reshape(self.n_seqs, e)
            tab[:] = -1
            for i, s in enumerate(seqs):
                table.table_into(s.req, grp.table_index, tab[i].ctypes.data, e)
        return dict(q_start_host=q_start, seq_lens_host=seq_lens, start_host=[s.start for s in seqs],
                    slots_host=slots, max_q_len=max(counts), max_seq_len=max(seq_lens),
                    any_from_last=any(s.from_last for s in seqs))

    def _fill_decode(self, buf, seqs, pools, vocab_size, temperatures, uniforms) -> dict:
        """The same for a decode step (every sequence brings one token and wants its logits): whole arrays at once."""
        n = self.n_seqs
        ids = np.fromiter((0 if s.from_last else s.tokens[0] for s in seqs), dtype=np.int64, count=n)
        if ids.min() < 0 or ids.max() >= vocab_size:
            raise ValueError("token outside vocabulary")
        self.part(buf, 9)[:] = np.fromiter((1 if s.from_last else 0 for s in seqs), dtype=np.int32, count=n)
        starts = np.fromiter((s.start for s in seqs), dtype=np.int32, count=n)
        ramp = np.arange(n + 1, dtype=np.int32)
        self.part(buf, 0)[:] = ids
        self.part(buf, 1)[:] = starts
        self.part(buf, 2)[:] = ramp[:n]
        self.part(buf, 3)[:] = ramp
        self.part(buf, 4)[:] = starts + 1
        table = pools.table
        slots = [table.slot(s.req) for s in seqs]
        self.part(buf, 5)[:] = slots
        self.part(buf, 6)[:] = ramp[:n]
        self.part(buf, 10)[:] = slots
        fl = self.part(buf, 7).view(np.float32)
        fl[:] = 0.0 if temperatures is None else temperatures
        fl = self.part(buf, 8).view(np.float32)
        fl[:] = 0.0 if uniforms is None else uniforms
        for g, grp in enumerate(pools.paged_groups):
            e = self.entries[g]
            tab = self.part(buf, self.first_table + g)
            tab[:] = -1
            ptr = tab.ctypes.data
            for i, s in enumerate(seqs):
                table.table_into(s.req, grp.table_index, ptr + i * e * 4, e)
        seq_lens = (starts + 1).tolist()
        return dict(q_start_host=ramp.tolist(), seq_lens_host=seq_lens, start_host=starts.tolist(), slots_host=slots,
                    max_q_len=1, max_seq_len=max(seq_lens), any_from_last=any(s.from_last for s in seqs))

    def views(self, dev: torch.Tensor, status: torch.Tensor, host_facts: dict) -> StepBatch:
        p = lambda i, n=None: self.part(dev, i, n)  # noqa: E731
        return StepBatch(
            n_tokens=self.n_tokens, n_seqs=self.n_seqs, n_rows=self.n_rows, token_ids=p(0), positions=p(1),
            seq_index=p(2), q_start=p(3), seq_lens=p(4), slots=p(5), logit_rows=p(6, self.n_rows),
            temperatures=p(7, self.n_rows).view(torch.float32), uniforms=p(8, self.n_rows).view(torch.float32),
            from_last=p(9), row_slots=p(10, self.n_rows),
            block_tables=[p(self.first_table + g).view(self.n_seqs, self.entries[g]) for g in range(len(self.entries))],
            status=status, **host_facts)


def check_sequences(seqs: list) -> None:
    if not seqs or sum(len(s.tokens) for s in seqs) == 0:
        raise ValueError("a step needs at least one token")
    for s in seqs:
        if not s.tokens:
            raise ValueError(f"request {s.req!r} brings no tokens to the step")


def build_batch(seqs: list, pools, device, status: torch.Tensor, vocab_size: int, temperatures=None,
                uniforms=None) -> StepBatch:
    """Lay out the metadata of ``seqs`` in one pinned buffer and copy it to the device."""
    check_sequences(seqs)
    longest = max(s.start + len(s.tokens) for s in seqs)
    entries = [max(1, -(-longest // pools.page_size)) for _ in pools.paged_groups]
    layout = BatchLayout(sum(len(s.tokens) for s in seqs), len(seqs), sum(len(s.want) for s in seqs), entries)
    host = torch.empty(layout.total, dtype=torch.int32, pin_memory=torch.cuda.is_available())
    facts = layout.fill(host.numpy(), seqs, pools, vocab_size, temperatures, uniforms)
    dev = host.to(device, non_blocking=True)
    return layout.views(dev, status, facts)
