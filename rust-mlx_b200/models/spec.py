"""What an architecture's ``build`` returns: parts and the order in which they run."""
from __future__ import annotations

from dataclasses import dataclass, field

from ..parts.base import LayerCall, Part


@dataclass
class ModelSpec(Part):
    """embedding -> blocks in ``schedule`` order -> final_norm -> head.

    ``schedule`` is data: a list of ``LayerCall(layer, cache)``.  ``ignored_tensors``
    are name patterns (fnmatch) that a checkpoint may hold without being an error."""

    config: object = None
    embedding: Part = None
    blocks: list = field(default_factory=list)
    schedule: list = field(default_factory=list)
    final_norm: Part = None
    head: Part = None
    ignored_tensors: tuple = ()
    vocab_size: int = 0
    eos_token_ids: tuple = ()

    graph_safe = True

    def children(self) -> list:
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def all_parts(self) -> list:
        out, todo = [], [self]
        while todo:
            part = todo.pop()
            out.append(part)
            todo.extend(part.children())
        return out

    def cache_specs(self) -> dict:
        """cache id -> CacheSpec of the run that writes it (the first that names it).  The block says what it
        remembers (``cache_specs()``); the schedule entry names one id for each."""
        out = {}
        for call in self.schedule:
            for cid, spec in zip(call.cache_ids(), self.blocks[call.layer].cache_specs()):
                out.setdefault(cid, spec)
        return out

    def check_schedule(self) -> None:
        writer = {}
        for call in self.schedule:
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"schedule names layer {call.layer}, the model has {len(self.blocks)}")
            specs, ids = self.blocks[call.layer].cache_specs(), call.cache_ids()
            # (a block that remembers nothing may still be given an id: it is not used)
            if specs and len(ids) != len(specs):
                raise ValueError(f"layer {call.layer} remembers {len(specs)} things, its schedule entry names "
                                 f"{len(ids)} caches")
            if len(set(ids)) != len(ids):
                raise ValueError(f"the schedule entry of layer {call.layer} names a cache twice")
            for cid, spec in zip(ids, specs):
                if cid in writer:
                    first = writer[cid][1]
                    if spec.group_key() != first.group_key():
                        raise ValueError(f"layer {call.layer} cannot read cache {cid}: its needs differ "
                                         f"from those of layer {writer[cid][0]} which writes it")
                else:
                    writer[cid] = (call.layer, spec)


def default_schedule(n_layers: int) -> list:
    return [LayerCall(i, i) for i in range(n_layers)]
