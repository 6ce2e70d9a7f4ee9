"""One step's batch: a flat list of tokens from several requests and what kernels
need to know about them, uploaded to the device in a single copy.

Per token: its id, its absolute position and the index of its sequence in the
batch.  Per sequence: where its tokens start in the flat list (``q_start``), its
length after this step (``seq_lens``), its state slot, and per paged cache group
its block table.  ``logit_rows`` are the flat indices of the tokens whose logits
are wanted.  The reference runs either one request's tokens or several requests'
single tokens at one offset (src/dense.rs:371, src/batching.rs:34-53); here any mix
is one batch.
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
    q_start_host: list
    seq_lens_host: list
    start_host: list
    slots_host: list
    max_q_len: int
    max_seq_len: int

    @property
    def all_decode(self) -> bool:
        return self.max_q_len == 1


def build_batch(seqs: list, pools, device, status: torch.Tensor, vocab_size: int) -> StepBatch:
    """Lay out the metadata of ``seqs`` in one pinned buffer and copy it to the device."""
    n_seqs = len(seqs)
    counts = [len(s.tokens) for s in seqs]
    n_tokens = sum(counts)
    if n_tokens == 0:
        raise ValueError("a step needs at least one token")
    rows = []
    q_start = [0]
    for s, c in zip(seqs, counts):
        if c == 0:
            raise ValueError(f"request {s.req!r} brings no tokens to the step")
        for w in s.want:
            if not 0 <= w < c:
                raise ValueError(f"request {s.req!r} wants logits at place {w} of {c} tokens")
            rows.append(q_start[-1] + w)
        q_start.append(q_start[-1] + c)
    n_rows = len(rows)
    table = pools.table
    groups = pools.paged_groups
    entries = [max(1, -(-max(s.start + c for s, c in zip(seqs, counts)) // pools.page_size)) for _ in groups]

    sizes = [n_tokens, n_tokens, n_tokens, n_seqs + 1, n_seqs, n_seqs, max(n_rows, 1)] + [n_seqs * e for e in entries]
    offsets = np.concatenate([[0], np.cumsum(sizes)])
    host = torch.empty(int(offsets[-1]), dtype=torch.int32, pin_memory=torch.cuda.is_available())
    buf = host.numpy()
    ids = np.fromiter((t for s in seqs for t in s.tokens), dtype=np.int64, count=n_tokens)
    if ids.min() < 0 or ids.max() >= vocab_size:
        raise ValueError("token outside vocabulary")
    buf[offsets[0]:offsets[1]] = ids
    pos = buf[offsets[1]:offsets[2]]
    sidx = buf[offsets[2]:offsets[3]]
    for i, (s, c) in enumerate(zip(seqs, counts)):
        pos[q_start[i]:q_start[i + 1]] = np.arange(s.start, s.start + c, dtype=np.int32)
        sidx[q_start[i]:q_start[i + 1]] = i
    buf[offsets[3]:offsets[4]] = q_start
    seq_lens = [s.start + c for s, c in zip(seqs, counts)]
    buf[offsets[4]:offsets[5]] = seq_lens
    slots_host = [table.slot(s.req) for s in seqs]
    buf[offsets[5]:offsets[6]] = slots_host
    buf[offsets[6]:offsets[7]] = rows if rows else [0]
    for g, grp in enumerate(groups):
        e = entries[g]
        tab = buf[offsets[7 + g]:offsets[8 + g]].reshape(n_seqs, e)
        tab[:] = -1
        for i, s in enumerate(seqs):
            table.table_into(s.req, grp.table_index, tab[i].ctypes.data, e)
    dev = host.to(device, non_blocking=True)

    def part(i, n=None):
        return dev[int(offsets[i]):int(offsets[i]) + (sizes[i] if n is None else n)]

    return StepBatch(
        n_tokens=n_tokens, n_seqs=n_seqs, n_rows=n_rows, token_ids=part(0), positions=part(1), seq_index=part(2),
        q_start=part(3), seq_lens=part(4), slots=part(5), logit_rows=part(6, n_rows),
        block_tables=[part(7 + g).view(n_seqs, entries[g]) for g in range(len(groups))], status=status,
        q_start_host=q_start, seq_lens_host=seq_lens, start_host=[s.start for s in seqs], slots_host=slots_host,
        max_q_len=max(counts), max_seq_len=max(seq_lens))
