"""The tensors behind the cache manager: page pools and state slots, in groups.

Caches (one per schedule cache id) with equal needs form a group: a paged group
has one pool of keys and one of values, [caches, pages, kv_heads, page_size,
head_dim] — inside a page each kv head's slots are contiguous, so one head's
keys of a page are one block of memory — and one block table per request; a
state group has [caches, slots, *state_shape].  A mixer sees its cache through
a view: its own slice of the pools and the batch's tables or slots.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..parts.base import CacheSpec
from .page_table import GroupGeometry, PageTable

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class PagedView:
    """What an attention mixer gets: pools of its cache and the batch's block tables."""

    k_pool: torch.Tensor       # [pages, kv_heads, page_size, head_dim]
    v_pool: torch.Tensor
    block_table: torch.Tensor  # int32 [sequences, entries], -1 where no page
    page_size: int
    window: int
    read_only: bool = False
    kind: str = "paged"


@dataclass
class StateView:
    """What a mixer with state of fixed size gets: [slots, *state_shape] and the batch's slots."""

    state: torch.Tensor
    slots: torch.Tensor        # int32 [sequences] on the device
    slots_host: list = field(default_factory=list)
    read_only: bool = False
    kind: str = "state"


@dataclass
class _Group:
    spec: CacheSpec
    cache_ids: list
    table_index: int = -1      # index among the paged groups of the page table, -1 for state groups
    k_pool: Optional[torch.Tensor] = None
    v_pool: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None


class CachePools:
    """Groups, their tensors and the page table for one model on one device."""

    def __init__(self, cache_specs: dict, *, max_tokens: int, page_size: int, max_requests: int,
                 dtype: torch.dtype, device):
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.groups = []
        self._where = {}  # cache id -> (group index, index inside the group)
        by_key = {}
        for cid in sorted(cache_specs):
            spec = cache_specs[cid]
            key = spec.group_key()
            if key not in by_key:
                by_key[key] = len(self.groups)
                self.groups.append(_Group(spec, []))
            g = by_key[key]
            self._where[cid] = (g, len(self.groups[g].cache_ids))
            self.groups[g].cache_ids.append(cid)
        geometry = []
        num_pages = -(-int(max_tokens) // self.page_size)
        for grp in self.groups:
            n = len(grp.cache_ids)
            if grp.spec.kind == "paged":
                grp.table_index = len(geometry)
                geometry.append(GroupGeometry(num_pages, self.page_size, grp.spec.window))
                shape = (n, num_pages, grp.spec.kv_heads, self.page_size, grp.spec.head_dim)
                grp.k_pool = torch.zeros(shape, dtype=dtype, device=device)
                grp.v_pool = torch.zeros(shape, dtype=dtype, device=device)
            elif grp.spec.kind == "state":
                sd = _STATE_DTYPES[grp.spec.state_dtype]
                grp.state = torch.zeros((n, self.max_requests, *grp.spec.state_shape), dtype=sd, device=device)
            else:
                raise ValueError(f"unknown cache kind {grp.spec.kind!r}")
        self.paged_groups = [g for g in self.groups if g.spec.kind == "paged"]
        self.state_groups = [g for g in self.groups if g.spec.kind == "state"]
        self.table = PageTable(geometry, self.max_requests)
        self.num_pages = num_pages

    def open(self, req: int) -> int:
        """A new request: takes a slot and clears its state."""
        slot = self.table.open(req)
        for grp in self.state_groups:
            grp.state[:, slot].zero_()
        return slot

    def reset_state(self, slots: list) -> None:
        """The fixed-size state of ``slots`` starts from zero (on the current stream).  Whoever admits requests
        without ``open`` (the scheduler takes slots from the page table itself) calls this for every request whose
        first tokens are about to run."""
        if not slots or not self.state_groups:
            return
        index = torch.tensor(slots, dtype=torch.long, device=self.state_groups[0].state.device)
        for grp in self.state_groups:
            grp.state.index_fill_(1, index, 0)

    def view(self, cache_id: int, batch, read_only: bool):
        g, i = self._where[cache_id]
        grp = self.groups[g]
        if grp.spec.kind == "paged":
            return PagedView(grp.k_pool[i], grp.v_pool[i], batch.block_tables[grp.table_index], self.page_size,
                             grp.spec.window, read_only)
        return StateView(grp.state[i], batch.slots, batch.slots_host, read_only)

    def bytes_per_token(self) -> int:
        total = 0
        for grp in self.paged_groups:
            total += 2 * len(grp.cache_ids) * grp.spec.kv_heads * grp.spec.head_dim * grp.k_pool.element_size()
        return total
