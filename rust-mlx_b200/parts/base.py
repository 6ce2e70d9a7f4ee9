"""Interfaces that every part of a layer implements.

A model is an embedding, a list of blocks, a schedule that says in which order
the blocks run and which cache each run uses, a final norm and an output head.
A block is put together from a mixer, a feed-forward and norms; an attention
mixer takes a position encoding.  Every part is built from sizes and constants
only (no part sees a model configuration), declares the tensors it needs by
their checkpoint names, and is bound to them once they are on the device.

The reference holds the same split with concrete types: ``Attention`` with its
constants as fields (src/dense.rs:112-126), ``Mlp`` (272-299), the norms as bare
arrays in ``DenseLayer`` (300-305).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part needs.

    ``init`` names the recipe of the random-weights mode ("linear", "embedding":
    N(0, 0.02); "norm": 1 + N(0, 0.05); "zeros"; "ones").  ``keep`` says how the tensor is
    held on the device: "compute" follows the run's dtype (bfloat16 or float32),
    "float32" stays 32-bit whatever the run's dtype, "int32" is an integer table.  ``optional``: a
    checkpoint may leave the tensor out (the part then finds no entry of that name in ``bind``), as
    the reference adds a projection's bias only where a tensor ``<prefix>.bias`` exists
    (src/weights.rs:96); the random-weights mode always makes it.
    """

    name: str
    shape: tuple
    init: str = "linear"
    keep: str = "compute"
    optional: bool = False


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer needs to remember per request.

    kind "paged": keys and values per token, ``kv_heads`` x ``head_dim`` each, in
    pages; ``window`` > 0 means only the last ``window`` positions are ever read, so
    older pages can be given back.  kind "state": ``state_shape`` numbers of
    ``state_dtype`` per request, of fixed size, zero when a request starts.
    Layers with equal specs share a cache group (one page pool geometry, one block
    table per request).
    """

    kind: str
    kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    state_shape: tuple = ()
    state_dtype: str = "float32"

    def group_key(self) -> tuple:
        if self.kind == "paged":
            return ("paged", self.kv_heads, self.head_dim, self.window)
        return ("state", self.state_shape, self.state_dtype)


@dataclass
class BuildContext:
    """What ``bind`` gets besides the tensors: the device, the compute dtype and the ops."""

    device: torch.device
    dtype: torch.dtype
    ops: object
    workspace: object
    # ``tap(name, tensor)``, or None: while set, parts hand it their named intermediate tensors (buffers of the
    # workspace that later layers overwrite, so whoever listens copies).  Names a dense block gives: residual, norm1, qkv, q_rot,
    # attn_out, mixer_out, norm2, ffn_act, ffn_out (the reference compares such tensors by name with an oracle's
    # dump, src/bin/trace.rs:4-24).
    tap: object = None


@dataclass(frozen=True)
class DecodeShape:
    """What is known of a decode step (every sequence brings one token) before it is laid out: how many
    sequences (spare places of a padded graph included) and the longest sequence's length after the step."""

    n_seqs: int
    max_seq_len: int


class Part:
    """Base of mixers, feed-forwards, norms, position encodings, embeddings and heads.

    ``graph_safe``: the part's ``forward`` may be captured in a CUDA graph and replayed for
    later steps of the same shape: it launches the same kernels with the same addresses
    and takes everything that changes from step to step (positions, block tables, slots)
    from the batch's device tensors, never from its host-side lists.  Off unless a part
    says so; one part that is not keeps the whole model on plain launches."""

    graph_safe = False

    def graph_key(self, shape: DecodeShape) -> tuple:
        """What, besides the number of sequences, decides which kernels with which launch shapes this part's
        ``forward`` issues for a decode step of ``shape`` (an attention mixer: into how many blocks it splits the
        keys, which follows the longest sequence).  A captured step is replayed only for steps with equal keys
        of all parts.  Most parts launch the same whatever the lengths: the empty tuple."""
        return ()

    def cache_specs(self) -> list:
        """What this part and the parts under it remember per request: one ``CacheSpec`` for each cache that a
        schedule entry has to name for it, in a fixed order (a block of one attention mixer: one)."""
        return []

    def param_specs(self) -> list:
        return []

    def bind(self, tensors: dict, ctx: BuildContext) -> None:
        """Take this part's tensors (by the names of ``param_specs``) from ``tensors``."""
        self.ctx = ctx

    def children(self) -> list:
        return []

    def linear_weights(self) -> list:
        """The bound matrices this part multiplies activations with (for timing product kernels)."""
        return []

    def gate_up_weights(self) -> list:
        """Fused gate/up matrices in blocks of 64 rows (for timing the product with the SwiGLU epilogue)."""
        return []

    def all_param_specs(self) -> list:
        specs = list(self.param_specs())
        for c in self.children():
            specs.extend(c.all_param_specs())
        return specs

    def bind_all(self, tensors: dict, ctx: BuildContext) -> None:
        for c in self.children():
            c.bind_all(tensors, ctx)
        self.bind(tensors, ctx)


class Norm(Part):
    """``forward(h, delta) -> (h, x)``: adds ``delta`` (or nothing) to the 32-bit residual
    stream ``h`` in place and returns the normalised rows in the compute dtype."""

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor]):
        raise NotImplementedError

    def forward_rows(self, h, delta, rows):
        """The same for the rows ``rows`` (int32 indices) only; ``h`` is left as it is."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Gives the rotation table an attention mixer hands to its kernel:
    ``rotary_dim`` (0: no rotation) and ``inv_freq`` (float32, rotary_dim/2 entries)."""

    rotary_dim: int = 0
    inv_freq: Optional[torch.Tensor] = None
    score_scale: float = 1.0   # attention scores are multiplied with this on top of the mixer's own scale

    def angles(self, batch):
        """Optional: [tokens, rotary_dim] float32, cosines then sines of the step's positions, formed once per
        step (kept in ``batch.per_step``).  None: the kernel forms them from ``inv_freq``."""
        return None


class Mixer(Part):
    """``forward(x, batch, cache) -> y`` over the flat token batch ``x`` [tokens, width].

    ``cache_spec`` says what the mixer remembers per request (None: nothing);
    ``cache`` is the view of its cache group for this run of the layer: pools,
    block tables or state slots (see ``cache.views``).  ``cache.read_only`` is set
    when the schedule lets this run read a cache that another run writes."""

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def cache_specs(self) -> list:
        spec = self.cache_spec()
        return [] if spec is None else [spec]

    def forward(self, x: torch.Tensor, batch, cache):
        raise NotImplementedError


class FeedForward(Part):
    """``forward(x) -> y`` row by row: [tokens, width] -> [tokens, width]."""

    def forward(self, x: torch.Tensor, batch=None):
        raise NotImplementedError


@dataclass(frozen=True)
class LayerCall:
    """One entry of a model's schedule: run block ``layer`` with cache ``cache``.

    The first entry that names a cache writes it; a later entry with the same cache
    reads what the first wrote and writes nothing.  A block may appear in several
    entries (it then runs more than once with the same weights).  ``cache`` is one id,
    or a tuple of ids for a block that remembers several things (one id for each entry
    of the block's ``cache_specs()``, in that order; the block's ``forward`` then gets a
    tuple of views)."""

    layer: int
    cache: object

    def cache_ids(self) -> tuple:
        return tuple(self.cache) if isinstance(self.cache, (tuple, list)) else (self.cache,)
