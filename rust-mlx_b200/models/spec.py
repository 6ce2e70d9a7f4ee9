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
        """cache id -> CacheSpec of the run that writes it (the first that names it)."""
        out = {}
        for call in self.schedule:
            if call.cache not in out:
                spec = self.blocks[call.layer].mixer.cache_spec()
                if spec is not None:
                    out[call.cache] = spec
        return out

    def check_schedule(self) -> None:
        writer = {}
        for call in self.schedule:
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"schedule names layer {call.layer}, the model has {len(self.blocks)}")
            spec = self.blocks[call.layer].mixer.cache_spec()
            if call.cache in writer:
                first = self.blocks[writer[call.cache]].mixer.cache_spec()
                if spec is None or first is None or spec.group_key() != first.group_key():
                    raise ValueError(f"layer {call.layer} cannot read cache {call.cache}: its needs differ "
                                     f"from those of layer {writer[call.cache]} which writes it")
            else:
                writer[call.cache] = call.layer


def default_schedule(n_layers: int) -> list:
    return [LayerCall(i, i) for i in range(n_layers)]
