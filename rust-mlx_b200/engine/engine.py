"""The engine: a model on one GPU, its cache, and the step function.

``Engine.step`` takes a batch of (request, its next tokens) — portions of prompts
beside single decoded tokens, cut anywhere — runs only those tokens, as one
batch, against the cache that earlier steps left, and returns float32 logits at
the wanted places.  The reference's ``DenseModel::forward`` (src/dense.rs:371-397)
runs one request's tokens and returns logits of every position; its batched decode
needs all rows at one offset (src/batching.rs:34-53).

There is no CPU path: the engine needs a CUDA device and this package's kernels.
"""
from __future__ import annotations

import os
import sys
import time

import torch

from ..cache.page_table import OutOfPages
from ..cache.pools import CachePools
from ..kernels import ops as _ops
from ..parts.base import BuildContext
from ..registry import build_model_spec, load_config
from ..weights.loader import load_tensors
from ..weights.random_init import random_tensors
from .batch import SequenceInput, StepBatch, build_batch
from .workspace import Workspace

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


class EngineError(RuntimeError):
    pass


def _log(msg):
    print(f"[rust_mlx_b200] {msg}", file=sys.stderr, flush=True)


class Engine:
    """A model ready to step.

    ``model``: a folder with config.json and safetensors, or (with
    ``random_weights=True``) a typed configuration / a folder whose config.json alone
    is read.  ``max_tokens``: how many tokens the cache holds in all (rounded up to
    pages).  ``dtype``: "bfloat16" (serving kernels) or "float32" (every product,
    norm and softmax in true 32-bit).  ``tuning``: which bfloat16 products of few rows take this
    package's tcgen05 kernel: "auto" times it against the library's product on the model's own
    weights when the engine starts (shapes whose weights together hold ``tune_min_bytes``), so two
    starts may choose differently and differ in last bits; "measured" is a fixed rule and
    ``tuning_table()`` of an earlier engine pins that engine's choices: one checkpoint, one set of
    bits.  "all" and "none" are for comparisons.
    """

    def __init__(self, model, *, dtype: str = "bfloat16", random_weights: bool = False, seed: int = 0,
                 max_tokens: int = 8192, page_size: int = 64, max_requests: int = 256, device: str = "cuda:0",
                 max_context: int = 0, cuda_graphs: bool = True, verbose: bool = False, tuning="auto",
                 tune_min_bytes: float = 256e6):
        if dtype not in _DTYPES:
            raise EngineError(f"dtype must be one of {sorted(set(_DTYPES))}, got {dtype!r}")
        if not torch.cuda.is_available():
            raise EngineError("no CUDA device: this engine runs on an NVIDIA B200 only and has no CPU path")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        major, minor = torch.cuda.get_device_capability(self.device)
        if major != 10:
            raise EngineError(f"the kernels are built for sm_100a; this device is sm_{major}{minor}")
        self.dtype = _DTYPES[dtype]
        self.dtype_name = "bfloat16" if self.dtype == torch.bfloat16 else "float32"
        if page_size <= 0 or page_size & (page_size - 1):
            raise EngineError(f"page_size must be a power of two, got {page_size}")
        t0 = time.time()
        _ops.kernels_library()  # builds at first use; raises if the extension cannot be had
        folder = None
        if isinstance(model, (str, os.PathLike)):
            folder = os.fspath(model)
            self.config = load_config(folder)
        else:
            self.config = model
        self.spec = build_model_spec(self.config)
        self.workspace = Workspace(self.device)
        self.ops = _ops.Kernels(tuning)     # this engine's switches and tuning results
        ctx = BuildContext(self.device, self.dtype, self.ops, self.workspace)
        self._ctx = ctx
        specs = self.spec.all_param_specs()
        if random_weights:
            tensors = random_tensors(specs, seed, self.dtype, self.device)
        else:
            if folder is None:
                raise EngineError("a model folder is needed unless random_weights is set")
            progress = (lambda i, n, name: _log(f"loaded {i}/{n} tensors") if i % 64 == 0 else None) if verbose else None
            tensors = load_tensors(folder, specs, self.dtype, self.device, self.spec.ignored_tensors, progress)
        self.spec.bind_all(tensors, ctx)
        del tensors
        self.vocab_size = self.spec.vocab_size
        self.page_size = page_size
        self.pools = CachePools(self.spec.cache_specs(), max_tokens=max_tokens, page_size=page_size,
                                max_requests=max_requests, dtype=self.dtype, device=self.device)
        # which schedule entry writes each cache: the first that names it.  An entry runs with one view for each thing
        # its block remembers: (cache id, whether this run only reads it)
        seen = set()
        self._calls = []
        for call in self.spec.schedule:
            ids = call.cache_ids()[:len(self.spec.blocks[call.layer].cache_specs())]
            self._calls.append((call, tuple((cid, cid in seen) for cid in ids)))
            seen.update(ids)
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # the token the last sampling chose for the request in each state slot: a decode step launched before the
        # host has read the step before takes its ids from here
        # (one word more than there are slots: the spare places of a padded decode graph leave their choice there)
        self.last_tokens = torch.zeros(max_requests + 1, dtype=torch.int32, device=self.device)
        # the longest sequence a request may reach: the cache's size, the model's stated limit, or the caller's
        limit = self.pools.num_pages * page_size
        stated = getattr(self.config, "max_position_embeddings", 0) or 0
        if stated > 0:
            limit = min(limit, stated)
        self.max_context = min(limit, max_context) if max_context > 0 else limit
        self._launches_per_graph = {}
        from .graphs import DecodeGraphs
        self.graphs = DecodeGraphs(self) if cuda_graphs and all(p.graph_safe for p in self.spec.all_parts()) else None
        self._req_ids = {}
        self._next_id = 0
        if self.dtype == torch.bfloat16 and self.ops.tcgen05_policy == "auto":
            weights = [w for part in self.spec.all_parts() for w in part.linear_weights()]
            self.ops.autotune_linears(weights, self.workspace, log=_log if verbose else None, min_bytes=tune_min_bytes)
            fused = [w for part in self.spec.all_parts() for w in part.gate_up_weights()]
            self.ops.autotune_fused_swiglu(fused, self.workspace, log=_log if verbose else None, min_bytes=tune_min_bytes)
        self.load_seconds = time.time() - t0
        if verbose:
            _log(f"model ready in {self.load_seconds:.1f}s: {len(self.spec.blocks)} layers, {self.dtype_name}, "
                 f"{self.pools.num_pages} pages of {page_size}")

    # ------------------------------------------------------------------ requests
    def _rid(self, key) -> int:
        rid = self._req_ids.get(key)
        if rid is None:
            rid = self._next_id
            self._next_id += 1
            self._req_ids[key] = rid
        return rid

    def length(self, key) -> int:
        """Tokens of request ``key`` in the cache (0 if it is not live)."""
        rid = self._req_ids.get(key)
        if rid is None or not self.pools.table.has(rid):
            return 0
        return self.pools.table.length(rid)

    def release(self, key) -> None:
        """The request is finished: its pages and its slot are given back."""
        rid = self._req_ids.pop(key, None)
        if rid is not None and self.pools.table.has(rid):
            self.pools.table.close(rid)

    # ------------------------------------------------------------------ the step
    def step(self, entries: list, end=()) -> torch.Tensor:
        """Run one batch.  ``entries``: (request, tokens, want) triples; ``want`` lists the
        places among these tokens whose logits are asked for.  Returns float32 logits
        [wanted, vocab] on the device, in the order of the entries and of ``want``.
        Requests in ``end`` are released after the step.  Raises ``OutOfPages`` (and
        changes nothing) if the cache cannot hold the step's tokens."""
        table = self.pools.table
        seqs, opened, grown = [], [], []
        try:
            keys = set()
            for key, tokens, want in entries:
                if key in keys:
                    raise EngineError(f"request {key!r} appears twice in one step")
                keys.add(key)
                if any((not isinstance(t, int)) or t < 0 or t >= self.vocab_size for t in tokens):
                    raise ValueError(f"request {key!r}: token outside vocabulary")
            for key, tokens, want in entries:
                rid = self._rid(key)
                if not table.has(rid):
                    self.pools.open(rid)
                    opened.append((key, rid))
                start = table.length(rid)
                table.reserve(rid, start + len(tokens))
                seqs.append(SequenceInput(rid, start, list(tokens), list(want)))
            batch = build_batch(seqs, self.pools, self.device, self._status, self.vocab_size)
        except Exception:
            for s in seqs:
                table.release_reserved(s.req)
            for key, rid in opened:
                table.close(rid)
                self._req_ids.pop(key, None)
            raise
        logits = self.forward(batch)
        self.check_status()
        for s in seqs:
            table.commit(s.req, s.start + len(s.tokens))
        for key in end:
            self.release(key)
        return logits.clone()  # the caller's own: the workspace buffer is written again by the next step

    def forward(self, batch: StepBatch) -> torch.Tensor:
        """The model over one batch whose pages are reserved: embedding, the schedule's
        layer runs, then final norm and head on the wanted rows."""
        spec = self.spec
        batch.per_step.clear()
        batch.last_tokens = self.last_tokens
        h = spec.embedding.forward(batch.token_ids, batch)
        pending = None
        for index, (call, caches) in enumerate(self._calls):
            views = tuple(self.pools.view(cid, batch, read_only) for cid, read_only in caches)
            self._run_index = index
            # a block that remembers one thing gets its view, one that remembers several a tuple of them
            cache = None if not views else (views[0] if len(views) == 1 else views)
            h, pending = spec.blocks[call.layer].forward(h, pending, batch, cache)
        if batch.n_rows == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        x = spec.final_norm.forward_rows(h, pending, batch.logit_rows)
        return spec.head.forward(x, batch)

    def step_with_intermediates(self, entries: list, end=()) -> tuple:
        """``step`` with every named intermediate tensor of every layer run copied out: returns (logits, {name:
        tensor}) with names ``run<i>.<name>`` for the i-th entry of the schedule, rows in the order of the
        step's tokens (what the reference's trace program compares with an oracle's dump by name,
        src/bin/trace.rs:4-24).  The kernels are the ones ``step`` runs."""
        taken = {}

        def tap(name, tensor):
            taken[f"run{self._run_index}.{name}"] = tensor.detach().clone()
        self._ctx.tap = tap
        try:
            logits = self.step(entries, end)
        finally:
            self._ctx.tap = None
        return logits, taken

    def generate(self, prompts: list, **options):
        """Token ids in, token ids out: see ``engine.generate.generate``.  Returns the list of
        generated ids per prompt."""
        from .generate import generate
        return generate(self, prompts, **options).tokens

    def generate_detailed(self, prompts: list, **options):
        from .generate import generate
        return generate(self, prompts, **options)

    def tuning_table(self) -> dict:
        """What this engine's tuning chose; ``Engine(..., tuning=table)`` makes the same choices again."""
        return self.ops.tuning_table()

    def check_status(self) -> None:
        """Kernels report what they could not do (a token without a page) in a status word."""
        code = int(self._status.item())
        if code != 0:
            self._status.zero_()
            what = {1: "a key was to be written to a position without a page",
                    2: "a key was to be read from a position without a page",
                    3: "a matrix product gave up waiting for its own copies or tensor-core operations"}.get(code, f"code {code}")
            raise EngineError(f"a kernel refused its input: {what}")
