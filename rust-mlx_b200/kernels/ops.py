"""Python faces of the CUDA kernels.

Every function takes torch tensors on the CUDA device, checks what the kernel
assumes (device, dtype, contiguity), and launches on torch's current stream.
There is no CPU path: a tensor that is not on a CUDA device is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from .library import KernelError, check, kernels_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

# how many launches of this package's kernels were made (bench reports it)
launch_count = 0


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {t.dtype}: kernels take float32 and bfloat16") from None


def _ptr(t, dtype=None, name="tensor"):
    if t is None:
        return c_void_p(0)
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}: kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return c_void_p(t.data_ptr())


def _stream():
    """The current stream of the current device as the kernels' void* (the raw handle: this runs once per launch)."""
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _launched(n=1):
    global launch_count
    launch_count += n


def count_launches(n: int) -> None:
    """Kernels of this package launched by replaying a captured graph."""
    _launched(n)


def embedding(ids, table, h_out, from_last=None, seq_index=None, slots=None, last_tokens=None):
    """h_out[t] = table[ids[t]] as float32 (the residual stream).  Where from_last[t] is set the id is the one the
    last step's sampling left for the token's sequence: last_tokens[slots[seq_index[t]]]."""
    lib = kernels_library()
    n, width = h_out.shape
    check(lib.rmx_embedding(_ptr(ids, torch.int32, "ids"), _ptr(table, name="table"), _ptr(h_out, torch.float32, "h"),
                            c_int(n), c_int(width), c_int(table.shape[0]), _ptr(from_last, torch.int32, "from_last"),
                            _ptr(seq_index, torch.int32, "seq_index"), _ptr(slots, torch.int32, "slots"),
                            _ptr(last_tokens, torch.int32, "last_tokens"), c_int(dtype_code(table)), _stream()))
    _launched()


def add_rmsnorm(h, delta, weight, eps, x_out, rows=None, write_h=True):
    """v = h + delta; h = v (if write_h); x_out = RMSNorm(v; weight, eps).  With ``rows`` the
    rows rows[r] are read, x_out[r] is written and h is left alone."""
    lib = kernels_library()
    n = x_out.shape[0]
    width = h.shape[1]
    if delta is not None and delta.dtype != x_out.dtype:
        raise KernelError("add_rmsnorm: delta and output must have the same dtype")
    check(lib.rmx_add_rmsnorm(_ptr(h, torch.float32, "h"), _ptr(delta, name="delta"), _ptr(rows, torch.int32, "rows"),
                              _ptr(weight, torch.float32, "weight"), c_float(eps), _ptr(x_out, name="x"),
                              c_int(n), c_int(width), c_int(1 if (write_h and rows is None) else 0),
                              c_int(dtype_code(x_out)), _stream()))
    _launched()


def add_residual(h, delta):
    lib = kernels_library()
    check(lib.rmx_add_residual(_ptr(h, torch.float32, "h"), _ptr(delta, name="delta"), c_int(h.shape[0]),
                               c_int(h.shape[1]), c_int(dtype_code(delta)), _stream()))
    _launched()


def add_bias(x, bias):
    """x[t, :] += bias in place (float add, one rounding).  ``x`` may be a view of some columns of wider rows."""
    lib = kernels_library()
    if x.dim() != 2 or x.stride(1) != 1 or bias.shape != (x.shape[1],) or not x.is_cuda:
        raise KernelError("add_bias: x must be [rows, width] with unit column stride on a CUDA device, bias [width]")
    check(lib.rmx_add_bias(c_void_p(x.data_ptr()), _ptr(bias, torch.float32, "bias"), c_int(x.shape[0]), c_int(x.shape[1]),
                           c_int(x.stride(0)), c_int(dtype_code(x)), _stream()))
    _launched()


def swiglu(gate_up, out, block=0):
    """out = silu(gate) * up.  A row of ``gate_up`` is [gate | up] (block 0) or blocks of ``block``
    gate numbers each followed by its ``block`` up numbers."""
    lib = kernels_library()
    n, inter = out.shape
    if gate_up.shape != (n, 2 * inter) or gate_up.dtype != out.dtype:
        raise KernelError("swiglu: gate_up must be [tokens, 2 * inter] of the output's dtype")
    check(lib.rmx_swiglu(_ptr(gate_up, name="gate_up"), _ptr(out, name="out"), c_int(n), c_int(inter), c_int(block),
                         c_int(dtype_code(out)), _stream()))
    _launched()


def gemm_plain(a, w, out):
    """out[M, N] = a[M, K] . w[N, K]^T on the FMA units, k in ascending order."""
    lib = kernels_library()
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n) or a.dtype != w.dtype:
        raise KernelError(f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not fit")
    check(lib.rmx_gemm_plain(_ptr(a, name="a"), _ptr(w, name="w"), _ptr(out, name="out"), c_int(m), c_int(n), c_int(k),
                             c_int(k), c_int(k), c_int(n), c_int(dtype_code(a)), c_int(dtype_code(out)), _stream()))
    _launched()


def rope_table(positions, inv_freq, rotary_dim, out):
    """out[t] = [cos(pos_t * inv_freq[j]) for j | sin(...) for j]: the angles of a step's positions, formed once."""
    lib = kernels_library()
    n = positions.shape[0]
    check(lib.rmx_rope_table(_ptr(positions, torch.int32, "positions"), _ptr(inv_freq, torch.float32, "inv_freq"),
                             _ptr(out, torch.float32, "out"), c_int(n), c_int(rotary_dim), _stream()))
    _launched()


def qk_rope_cache(qkv, q_norm, k_norm, eps, inv_freq, rotary_dim, positions, seq_index, block_table, page_size,
                  k_pool, v_pool, q_out, nq, nkv, hd, write_kv, status, cos_sin=None):
    lib = kernels_library()
    n = qkv.shape[0]
    check(lib.rmx_qk_rope_cache(
        _ptr(qkv, name="qkv"), _ptr(q_norm, torch.float32, "q_norm"), _ptr(k_norm, torch.float32, "k_norm"),
        c_float(eps), _ptr(inv_freq, torch.float32, "inv_freq"), c_int(rotary_dim),
        _ptr(positions, torch.int32, "positions"), _ptr(seq_index, torch.int32, "seq_index"),
        _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size),
        _ptr(k_pool, qkv.dtype, "k_pool"), _ptr(v_pool, qkv.dtype, "v_pool"), _ptr(q_out, qkv.dtype, "q_out"),
        c_int(n), c_int(nq), c_int(nkv), c_int(hd), c_int(qkv.shape[1]), c_int(1 if write_kv else 0),
        _ptr(status, torch.int32, "status"), _ptr(cos_sin, torch.float32, "cos_sin"), c_int(dtype_code(qkv)), _stream()))
    _launched()


def attention_plain(q, k_pool, v_pool, positions, seq_index, block_table, page_size, out, nq, nkv, hd, window,
                    scale, status):
    lib = kernels_library()
    n = q.shape[0]
    check(lib.rmx_attention_plain(
        _ptr(q, name="q"), _ptr(k_pool, q.dtype, "k_pool"), _ptr(v_pool, q.dtype, "v_pool"),
        _ptr(positions, torch.int32, "positions"), _ptr(seq_index, torch.int32, "seq_index"),
        _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size),
        _ptr(out, q.dtype, "out"), c_int(n), c_int(nq), c_int(nkv), c_int(hd), c_int(window), c_float(scale),
        _ptr(status, torch.int32, "status"), c_int(dtype_code(q)), _stream()))
    _launched()


def sample(logits, temperature, uniform, out, slots=None, last_tokens=None):
    """out[r] = greedy choice (temperature None or 0) or a draw from softmax(logits / temperature); with ``slots``
    and ``last_tokens`` the choice is also left at last_tokens[slots[r]] for the next step's embedding."""
    lib = kernels_library()
    r, v = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("sample: logits rows must be contiguous")
    if not logits.is_cuda or logits.dtype != torch.float32:
        raise KernelError("sample: logits must be float32 on a CUDA device")
    check(lib.rmx_sample(c_void_p(logits.data_ptr()), c_int(logits.stride(0)), _ptr(temperature, torch.float32, "temperature"),
                         _ptr(uniform, torch.float32, "uniform"), _ptr(out, torch.int32, "out"), c_int(r), c_int(v),
                         _ptr(slots, torch.int32, "slots"), _ptr(last_tokens, torch.int32, "last_tokens"), _stream()))
    _launched()


# ---------------------------------------------------------------------------
# Helpers of the dispatch below that hold no state.

def _mpad(m: int) -> int:
    return 16 if m <= 16 else (32 if m <= 32 else 64)


def _graph_time(fn, calls: int, reps: int = 3) -> float:
    """Microseconds per call of ``fn(i)``, timed on the device inside a captured graph."""
    fn(0)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(calls):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        g.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / reps / calls * 1e3


class _Sequences:
    """A run of neighbouring sequences of a batch, with what the attention kernels read of a batch.  Token
    numbers in ``q_start`` stay those of the whole batch, so q, out and positions are passed whole."""

    def __init__(self, batch, first: int, last: int):
        self.q_start = batch.q_start[first:last + 1]
        self.q_start_host = batch.q_start_host[first:last + 1]
        self.n_seqs = last - first
        lens = batch.seq_lens_host[first:last]
        counts = [self.q_start_host[i + 1] - self.q_start_host[i] for i in range(self.n_seqs)]
        self.max_seq_len, self.max_q_len = max(lens), max(counts)
        self.positions, self.status = batch.positions, batch.status
        self.first, self.last = first, last


def _short_and_long(batch, group: int):
    """A mixed step: decoded tokens (rows * group <= 16: the key-split kernel's case) beside prompt portions.  If
    the short sequences are the batch's head or its tail, returns the two runs (short, long), else None."""
    if getattr(batch, "seq_lens_host", None) is None or batch.n_seqs < 2:
        return None
    key = ("short_and_long", group)
    memo = getattr(batch, "per_step", None)
    if memo is not None and key in memo:
        return memo[key]
    starts = batch.q_start_host
    short = [(starts[i + 1] - starts[i]) * group <= 16 for i in range(batch.n_seqs)]
    n_short = sum(short)
    found = None
    if 0 < n_short < batch.n_seqs:
        if all(short[:n_short]):
            found = (_Sequences(batch, 0, n_short), _Sequences(batch, n_short, batch.n_seqs))
        elif all(short[batch.n_seqs - n_short:]):
            found = (_Sequences(batch, batch.n_seqs - n_short, batch.n_seqs), _Sequences(batch, 0, batch.n_seqs - n_short))
    if memo is not None:
        memo[key] = found
    return found


def flash_supported(hd: int, group: int) -> bool:
    return bool(kernels_library().rmx_attention_flash_supports(c_int(hd), c_int(group)))


_SM_COUNT = None


def _sm_count() -> int:
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _SM_COUNT


def flash_splits(n_tiles: int, nkv: int, max_seq_len: int) -> int:
    """Few rows and long contexts (decoding): share a tile's keys among blocks so that every
    SM has work.  Up to 8 splits form a thread-block cluster and add their results through shared
    memory, which costs far less than the round through global memory that more splits take.
    Measured on B200 at 8 kv heads: clusters of 2, 4 and 8 are placed readily, of 3 or 6 not; the
    grid should stay a little under two blocks per SM, which the kernels before and after need
    some of; and 4 splits beat 8 as soon as 4 give 128 blocks.  So: the largest of 1, 2, 4, 8 that
    keeps the grid under 7/8 of two blocks per SM, 4 rather than 8 if 4 give 128 blocks; more than
    8 only where each split still has 16 tiles of 64 keys."""
    blocks = n_tiles * nkv
    kv_tiles = -(-max_seq_len // 64)
    room = 2 * _sm_count() - _sm_count() // 4
    if blocks >= room or kv_tiles < 4:
        return 1
    want = max(1, min(room // blocks, kv_tiles // 2, 64))
    if want > 8 and kv_tiles // want >= 16 and blocks * 8 < 128:
        return want
    splits = 8 if want >= 8 else (4 if want >= 4 else (2 if want >= 2 else 1))
    if splits == 8 and blocks * 4 >= 128:
        splits = 4
    return splits


def flash_takes_projection(hd: int, group: int, page_size: int, rotary_dim: int) -> bool:
    """Whether the key-split kernel is built to finish the q/k/v projection of a decoding step at these sizes."""
    return bool(kernels_library().rmx_attention_flash_takes_projection(c_int(hd), c_int(group), c_int(page_size), c_int(rotary_dim)))


def attention_flash(q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace,
                    n_splits=None, projection=None, use_tma=True):
    """Tensor-core attention over pages for bfloat16 (prompt portions and decoded tokens alike).  ``projection``:
    (qkv rows, q_norm, k_norm, eps, cos_sin, write_kv) for a decoding step whose kernel finishes the projection.
    ``use_tma``: keys and values are fetched by TMA where the kernel is built for it."""
    lib = kernels_library()
    group = nq // nkv
    tq = 64 // group
    starts = batch.q_start_host
    n_tiles = sum(-(-(starts[i + 1] - starts[i]) // tq) for i in range(batch.n_seqs))
    if n_splits is None:
        n_splits = flash_splits(n_tiles, nkv, batch.max_seq_len)
    n = out.shape[0]
    qkv, q_norm, k_norm, eps, cos_sin, write_kv = projection if projection is not None else (None, None, None, 0.0, None, False)
    part_o = part_ml = counters = None
    if n_splits > 1:
        part_o = workspace.get("attn_part_o", (n_splits, n * nq, hd), torch.float32)
        part_ml = workspace.get("attn_part_ml", (n_splits, n * nq, 2), torch.float32)
        counters = workspace.get_zeroed("attn_counters", (max(4096, batch.n_seqs * nkv),), torch.int32)
    check(lib.rmx_attention_flash(
        _ptr(q if qkv is None else None, torch.bfloat16, "q"), _ptr(k_pool, torch.bfloat16, "k_pool"), _ptr(v_pool, torch.bfloat16, "v_pool"),
        _ptr(batch.q_start, torch.int32, "q_start"), _ptr(batch.positions, torch.int32, "positions"),
        _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size),
        _ptr(out, torch.bfloat16, "out"), _ptr(part_o), _ptr(part_ml), _ptr(counters), c_int(batch.n_seqs), c_int(n),
        c_int(n_tiles),
        c_int(nq), c_int(nkv), c_int(hd), c_int(window), c_float(scale), c_int(n_splits),
        c_int(getattr(batch, "max_q_len", 0)), c_int(k_pool.shape[0] if use_tma else 0),
        _ptr(qkv, torch.bfloat16, "qkv"), c_int(qkv.stride(0) if qkv is not None else 0), _ptr(q_norm, torch.float32, "q_norm"),
        _ptr(k_norm, torch.float32, "k_norm"), c_float(eps), _ptr(cos_sin, torch.float32, "cos_sin"), c_int(1 if write_kv else 0),
        c_int(starts[0]), c_int(starts[batch.n_seqs] - starts[0]), _ptr(batch.status, torch.int32, "status"), _stream()))
    _launched(2 if n_splits > 1 else 1)


_scratch = None


def _own_workspace():
    """Scratch for kernels called without an engine's workspace (tests, single calls)."""
    global _scratch
    if _scratch is None:
        from ..engine.workspace import Workspace
        _scratch = Workspace(torch.device("cuda", torch.cuda.current_device()))
    return _scratch


_supported = {}


def tcgen05_supported(m: int, n: int, k: int) -> bool:
    key = (m, n, k)
    if key not in _supported:
        if len(_supported) > 65536:
            _supported.clear()
        _supported[key] = bool(kernels_library().rmx_gemm_tcgen05_supports(c_int(m), c_int(n), c_int(k)))
    return _supported[key]


def tcgen05_splits(m: int, n: int, k: int) -> int:
    """How many slices of K share a tile of 128 weight rows.  The product is bound by reading the
    weight: what matters is that enough blocks are resident to keep loads in flight on every SM
    (measured on Qwen3-8B shapes), not that the last wave is full.  So: the fewest slices that
    give at least 128 blocks; as many as give 192 blocks where each slice then still has 24
    k-blocks of 64 (long reductions: the down projection); at most 8 (a cluster), each slice
    keeping at least 4 k-blocks."""
    tiles = -(-n // 128)
    k_blocks = -(-k // 64)
    if tiles >= 128:
        return 1
    splits = -(-128 // tiles)
    more = -(-192 // tiles)
    if more <= 8 and k_blocks // more >= 24:
        splits = more
    return max(1, min(splits, 8, k_blocks // 4))


def gemm_tcgen05(a, w, out, workspace=None, status=None, splits=None, cluster=True, dependent=False, swiglu=False):
    """out[M, N] = a[M, K] . w[N, K]^T for M <= 64 on the tcgen05 tensor cores (bfloat16 in,
    float accumulation, bfloat16 or float out).  ``cluster``: split-K slices of a tile form a
    thread-block cluster and add their sums through distributed shared memory (up to 8 slices),
    else through scratch in global memory.  ``dependent``: launch as a programmatic dependent of
    the kernel before it on the stream, so that its weight loads start while that kernel ends."""
    lib = kernels_library()
    m, k = a.shape
    n = w.shape[0]
    # swiglu: w's rows come in blocks of 64 gate rows and their 64 up rows; out is silu(gate) * up, [m, n / 2]
    want_shape = (m, n // 2) if swiglu else (m, n)
    if w.shape[1] != k or out.shape != want_shape or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tcgen05: {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} of {a.dtype}")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tcgen05: the result is bfloat16 or float32")
    ws = workspace if workspace is not None else _own_workspace()
    if splits is None:
        splits = tcgen05_splits(m, n, k)
        if cluster:
            splits = min(splits, 8)
    partial = counters = None
    if splits > 1:
        need = lib.rmx_gemm_tcgen05_scratch_floats(c_int(m), c_int(n), c_int(splits))
        partial = ws.get("gemm_partial", (need,), torch.float32)
        counters = ws.get_zeroed("gemm_counters", (max(4096, -(-n // 128)),), torch.int32)
    if status is None:
        status = ws.get_zeroed("gemm_status", (1,), torch.int32)
    check(lib.rmx_gemm_tcgen05(
        _ptr(a, name="a"), _ptr(w, name="w"), _ptr(out, name="out"), c_int(m), c_int(n), c_int(k), c_int(a.stride(0)),
        c_int(w.stride(0)), c_int(out.stride(0)), c_int(1 if out.dtype == torch.float32 else 0), c_int(splits),
        _ptr(partial), _ptr(counters), _ptr(status, torch.int32, "status"),
        c_int((1 if cluster else 0) | (2 if dependent else 0) | (4 if swiglu else 0)), _stream()))
    _launched()
    return status


def gemm_tcgen05_wait_probe(a, w, out, status, splits=1, cluster=True, swiglu=False, spin_limit=1000, workspace=None):
    """For tests: the tcgen05 product's kernel launched so that its waits run out (no tile is ever copied, every
    wait gives up after ``spin_limit`` polls).  It must return, leave status 3 in ``status`` and ``out`` untouched."""
    lib = kernels_library()
    m, k = a.shape
    n = w.shape[0]
    ws = workspace if workspace is not None else _own_workspace()
    partial = counters = None
    if splits > 1:
        partial = ws.get("gemm_partial", (lib.rmx_gemm_tcgen05_scratch_floats(c_int(m), c_int(n), c_int(splits)),), torch.float32)
        counters = ws.get_zeroed("gemm_counters", (max(4096, -(-n // 128)),), torch.int32)
    check(lib.rmx_gemm_tcgen05_wait_probe(
        _ptr(a, torch.bfloat16, "a"), _ptr(w, torch.bfloat16, "w"), _ptr(out, name="out"), c_int(m), c_int(n), c_int(k),
        c_int(a.stride(0)), c_int(w.stride(0)), c_int(out.stride(0)), c_int(1 if out.dtype == torch.float32 else 0),
        c_int(splits), _ptr(partial), _ptr(counters), _ptr(status, torch.int32, "status"),
        c_int((1 if cluster else 0) | (4 if swiglu else 0)), c_int(spin_limit), _stream()))
    _launched()
    return counters


def tcgen05_attention_supported(hd: int, group: int, page_size: int) -> bool:
    return bool(kernels_library().rmx_attention_tcgen05_supports(c_int(hd), c_int(group), c_int(page_size)))


def tcgen05_attention_shape(counts: list, nkv: int, group: int, max_seq_len: int) -> tuple:
    """(query tiles a block, runs of keys) for prompt portions of ``counts`` tokens.  Measured on 148 SMs: a grid of
    about one block an SM (not more) is fastest; two neighbouring tiles of 128 rows a block, which share the key and
    value tiles it fetches, win once a sequence has some 2,000 keys, one tile a block below that; where whole tiles
    leave SMs without work, every tile's keys go in as many runs as fill them (at most 8, each of at least 4 key
    tiles of 64), whose shares a second kernel adds."""
    tile = 128 // group
    sms = _sm_count()
    pairs = sum(-(-c // (2 * tile)) for c in counts) * nkv
    singles = sum(-(-c // tile) for c in counts) * nkv
    key_tiles = -(-max_seq_len // 64)
    if 4 * pairs >= 3 * sms:
        return 2, 1
    long_keys = max_seq_len >= 2048
    if 4 * singles >= 3 * sms:   # one tile a block would fill the SMs
        return (2, max(1, min(sms // pairs, 8, key_tiles // 4))) if long_keys else (1, 1)
    if long_keys:
        return 2, max(1, min(sms // pairs, 8, key_tiles // 4))
    return 1, max(1, min(sms // singles, 8, key_tiles // 4))


def attention_tcgen05(q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, per_block=None,
                      n_splits=None, workspace=None):
    """Prompt portions: S = Q K^T and O += P V as tcgen05 MMAs with accumulators in tensor memory (see
    ``tcgen05_attention_shape`` for how the work is divided; ``per_block`` and ``n_splits`` override it)."""
    lib = kernels_library()
    tile = 128 // (nq // nkv)
    starts = batch.q_start_host
    counts = [starts[i + 1] - starts[i] for i in range(batch.n_seqs)]
    if per_block is None and n_splits is None:
        per_block, n_splits = tcgen05_attention_shape(counts, nkv, nq // nkv, batch.max_seq_len)
        if workspace is None:
            n_splits = 1
    per_block = 2 if per_block is None else per_block
    n_splits = 1 if n_splits is None else n_splits
    n_tiles = sum(-(-c // (per_block * tile)) for c in counts)
    part_o = part_ml = None
    if n_splits > 1:
        ws = workspace if workspace is not None else _own_workspace()
        part_o = ws.get("attn_part_o", (n_splits, q.shape[0] * nq, hd), torch.float32)
        part_ml = ws.get("attn_part_ml", (n_splits, q.shape[0] * nq, 2), torch.float32)
    check(lib.rmx_attention_tcgen05(
        _ptr(q, torch.bfloat16, "q"), _ptr(k_pool, torch.bfloat16, "k_pool"), _ptr(v_pool, torch.bfloat16, "v_pool"),
        _ptr(batch.q_start, torch.int32, "q_start"), _ptr(batch.positions, torch.int32, "positions"),
        _ptr(block_table, torch.int32, "block_table"), c_int(block_table.shape[1]), c_int(page_size),
        _ptr(out, torch.bfloat16, "out"), c_int(batch.n_seqs), c_int(q.shape[0]), c_int(n_tiles), c_int(per_block),
        c_int(nq), c_int(nkv), c_int(hd), c_int(window), c_float(scale), c_int(k_pool.shape[0]), c_int(n_splits),
        _ptr(part_o), _ptr(part_ml), c_int(starts[0]), c_int(starts[-1] - starts[0]), _ptr(batch.status, torch.int32, "status"), _stream()))
    _launched(2 if n_splits > 1 else 1)


# Whether this package's kernels are launched as programmatic dependents of the kernel before them (a switch of the
# loaded library, so of the process: see ``set_dependent_launch``).
dependent_launch = True


def set_dependent_launch(on: bool) -> None:
    """Programmatic dependent launch of this package's kernels (on by default): a kernel's blocks may take their
    places while the kernel before it drains, and the tcgen05 product fetches weights meanwhile."""
    global dependent_launch
    dependent_launch = bool(on)
    kernels_library().rmx_set_dependent_launch(c_int(1 if on else 0))


# ---------------------------------------------------------------------------
# Dispatch: which kernel serves a call.  float32 always takes the plain kernels (fixed order of summation, no
# tensor cores); bfloat16 takes the fast ones where they apply.  The choices that can be switched or tuned belong
# to a ``Kernels`` object: every engine has its own and hands it to its parts, so two engines in one process
# neither share tuning results nor see each other's switches.

class Kernels:
    """The kernels as one engine sees them: its switches, what its tuning measured, and the dispatch that reads
    both.  Everything else (the plain faces of the kernels above) is reached through it by name.

    ``policy``: which products of few rows (up to 64) take this package's tcgen05 kernel rather than the library's
    product: "auto" (whichever was faster when the engine timed both on the model's own weights, see
    ``autotune_linears``; shapes that were not timed follow "measured"), "measured" (the output head and long
    reductions, where it won on Qwen3-8B shapes: a fixed rule, the same bits on every start), "all" (every product
    the kernel supports), "none"; or a table that ``tuning_table`` returned earlier (the choices of that run again).
    """

    def __init__(self, policy="measured"):
        self.tuned = {}          # (n, k, padded rows[, "swiglu"]) -> True if the tcgen05 kernel was faster
        self.tuned_splits = {}   # (n, k, padded rows) -> the number of K slices that was fastest
        if isinstance(policy, dict):
            self.load_tuning_table(policy)
            policy = "auto"
        if policy not in ("auto", "measured", "all", "none"):
            raise KernelError(f"unknown kernel policy {policy!r}: auto, measured, all, none or a tuning table")
        self.tcgen05_policy = policy
        self.use_tma = True                 # decoding fetches keys and values by TMA where the kernel is built for it
        self.fused_decode_rope = True       # a decoding attention norms and rotates its own token while it waits for keys
        self.fused_swiglu = True            # the gate/up product of few rows forms silu(gate) * up in its epilogue
        self.use_tcgen05_attention = True   # prompt portions at head size 128 run on the tcgen05 tensor cores
        self._splits_memo = {}

    def __getattr__(self, name):
        # the faces of the kernels that hold no state
        try:
            return globals()[name]
        except KeyError:
            raise AttributeError(name) from None

    @property
    def dependent_launch(self) -> bool:
        return dependent_launch

    # ---- tuning ---------------------------------------------------------------------------------------------
    def tuning_table(self) -> dict:
        """What the tuning chose, in a form that JSON takes and ``Kernels(policy=table)`` reads back."""
        key = lambda k: "x".join(str(p) for p in k)   # noqa: E731
        return {"policy": self.tcgen05_policy, "tcgen05": {key(k): bool(v) for k, v in sorted(self.tuned.items(), key=str)},
                "slices": {key(k): int(v) for k, v in sorted(self.tuned_splits.items(), key=str)}}

    def load_tuning_table(self, table: dict) -> None:
        def key(text):
            return tuple(int(p) if p.lstrip("-").isdigit() else p for p in text.split("x"))
        self.tuned = {key(k): bool(v) for k, v in (table.get("tcgen05") or {}).items()}
        self.tuned_splits = {key(k): int(v) for k, v in (table.get("slices") or {}).items()}

    def prefers_tcgen05(self, m: int, n: int, k: int) -> bool:
        if self.tcgen05_policy == "none" or not tcgen05_supported(m, n, k):
            return False
        if self.tcgen05_policy == "all":
            return True
        if self.tcgen05_policy == "auto" and (n, k, _mpad(m)) in self.tuned:
            return self.tuned[(n, k, _mpad(m))]
        return n * k >= (1 << 28) or (k >= 8192 and m <= 32)

    def autotune_linears(self, weights: list, workspace=None, rows=(8, 32, 64), log=None, min_bytes: float = 256e6) -> dict:
        """Time the tcgen05 product against the library's on the model's own bfloat16 weights, per
        shape and per padded row count, and remember the faster.  Weights of one shape take turns so
        that none is served from L2 (a lone small weight would be: its timing then says little and
        the rule of "measured" stands for it; ``min_bytes`` is how much a shape's weights must hold
        together to be timed)."""
        groups = {}
        for w in weights:
            if w is not None and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_cuda:
                groups.setdefault((w.shape[0], w.shape[1]), []).append(w)
        for (n, k), ws in groups.items():
            if not tcgen05_supported(1, n, k) or len(ws) * n * k * 2 < min_bytes:
                continue
            for m in rows:
                key = (n, k, _mpad(m))
                if key in self.tuned:
                    continue
                a = torch.randn(m, k, device=ws[0].device).to(torch.bfloat16)
                out = torch.empty(m, n, dtype=torch.bfloat16, device=ws[0].device)
                calls = max(4, min(len(ws), 12))
                # the kernel's own choice first: how many slices of K share a tile (from one less than the rule's count up to
                # what a cluster takes: more slices mean fewer k-blocks for each block to stream, and a longer reduction)
                most = 8
                rule = min(tcgen05_splits(m, n, k), most)
                best = None
                for splits in range(max(1, rule - 1), most + 1):
                    if splits > max(1, -(-k // 64) // 4):
                        continue
                    t = _graph_time(lambda i: gemm_tcgen05(a, ws[i % len(ws)], out, workspace, splits=splits, dependent=True), calls)
                    if best is None or t < best[0]:
                        best = (t, splits)
                mine, self.tuned_splits[key] = best
                lib = _graph_time(lambda i: torch.mm(a, ws[i % len(ws)].t(), out=out), calls)
                self.tuned[key] = mine < lib
                if log is not None:
                    log(f"product [{m} x {k}] . [{n} x {k}]^T: tcgen05 {mine:.1f} us with {best[1]} slices of K, library {lib:.1f} us")
        return dict(self.tuned)

    def autotune_fused_swiglu(self, weights: list, workspace=None, rows=(8, 32, 64), log=None, min_bytes: float = 256e6) -> dict:
        """The same for gate/up weights in blocks of 64: the tcgen05 product with the SwiGLU epilogue
        against the library's product followed by the pointwise kernel."""
        groups = {}
        for w in weights:
            if w is not None and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_cuda and w.shape[0] % 128 == 0:
                groups.setdefault((w.shape[0], w.shape[1]), []).append(w)
        for (n, k), ws in groups.items():
            if not tcgen05_supported(1, n, k) or len(ws) * n * k * 2 < min_bytes:
                continue
            for m in rows:
                key = (n, k, _mpad(m), "swiglu")
                if key in self.tuned:
                    continue
                a = torch.randn(m, k, device=ws[0].device).to(torch.bfloat16)
                gu = torch.empty(m, n, dtype=torch.bfloat16, device=ws[0].device)
                act = torch.empty(m, n // 2, dtype=torch.bfloat16, device=ws[0].device)
                calls = max(4, min(len(ws), 12))
                best = None
                for splits in range(1, 4):    # (a weight with this many tiles seldom gains from slices of K; it is asked, not assumed)
                    if splits > max(1, -(-k // 64) // 4):
                        continue
                    t = _graph_time(lambda i: gemm_tcgen05(a, ws[i % len(ws)], act, workspace, swiglu=True, splits=splits, dependent=True), calls)
                    if best is None or t < best[0]:
                        best = (t, splits)
                mine, self.tuned_splits[key] = best

                def lib_pair(i):
                    torch.mm(a, ws[i % len(ws)].t(), out=gu)
                    swiglu(gu, act, 64)
                lib = _graph_time(lib_pair, calls)
                # inside a step the fused product also spares a kernel's start and end, which this timing of the pair
                # alone does not show: it is taken unless the pair is clearly faster
                self.tuned[key] = mine < lib * 1.05
                if log is not None:
                    log(f"gate/up [{m} x {k}] . [{n} x {k}]^T + SwiGLU: fused tcgen05 {mine:.1f} us with {best[1]} slices of K, library + pointwise {lib:.1f} us")
        return dict(self.tuned)

    def prefers_fused_swiglu(self, m: int, n: int, k: int) -> bool:
        """The fused product saves a kernel and the round trip of the [m, n] intermediate; it is taken
        wherever the tcgen05 kernel runs at all, unless timing said the library's product plus the
        pointwise kernel is faster for this shape."""
        if not self.fused_swiglu or self.tcgen05_policy == "none" or not tcgen05_supported(m, n, k) or n % 128:
            return False
        return self.tuned.get((n, k, _mpad(m), "swiglu"), True)

    # ---- products -------------------------------------------------------------------------------------------
    def linear(self, x, w, out, workspace=None, status=None):
        """out = x . w^T.  w is [out_features, in_features] as stored in the checkpoint."""
        if x.dtype == torch.float32:
            gemm_plain(x, w, out)
        else:
            self.linear_bf16(x, w, out, workspace, status)

    def linear_bf16(self, x, w, out, workspace=None, status=None):
        """bfloat16 operands, float accumulation; the result in bfloat16 or (for logits) float32."""
        m, k = x.shape
        if self.prefers_tcgen05(m, w.shape[0], k) and x.stride(1) == 1 and w.stride(1) == 1:
            self.gemm_tcgen05(x, w, out, workspace, status, dependent=dependent_launch)
        elif out.dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
        else:
            torch.mm(x, w.t(), out_dtype=torch.float32, out=out)

    def gemm_tcgen05(self, a, w, out, workspace=None, status=None, splits=None, cluster=True, dependent=False, swiglu=False):
        """The tcgen05 product with the number of K slices that this engine's tuning found best for the shape."""
        if splits is None:
            key = (w.shape[0], a.shape[1], _mpad(a.shape[0])) + (("swiglu",) if swiglu else ())
            splits = self.tuned_splits.get(key)
            if splits is not None and cluster:
                splits = min(splits, 8)
        return gemm_tcgen05(a, w, out, workspace, status, splits, cluster, dependent, swiglu)

    # ---- attention ------------------------------------------------------------------------------------------
    def decode_takes_projection(self, batch, dtype, hd: int, group: int, page_size: int, rotary_dim: int, cos_sin) -> bool:
        """Whether this step's attention may be handed the q/k/v projection's rows as they come: every sequence brings
        one token, heads of 128 all rotated, bfloat16, pages the TMA kernel takes."""
        return (self.fused_decode_rope and self.use_tma and dtype == torch.bfloat16 and cos_sin is not None
                and getattr(batch, "max_q_len", 0) == 1 and batch.n_seqs == batch.positions.shape[0]
                and flash_takes_projection(hd, group, page_size, rotary_dim))

    def attention_flash(self, *args, **kwargs):
        kwargs.setdefault("use_tma", self.use_tma)
        return attention_flash(*args, **kwargs)

    def attention(self, q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace=None,
                  projection=None):
        """Picks the attention kernel for the dtype, head size and shape of the step.  A step that mixes decoded
        tokens with prompt portions runs as two launches, each kind with the kernel made for it.  ``projection``
        (see ``decode_takes_projection``): the q/k/v rows before norm and rotation, which the decoding kernel then
        finishes itself; ``q`` is not read."""
        group = nq // nkv
        if projection is not None:
            self.attention_flash(q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace,
                                 projection=projection)
            return
        if q.dtype == torch.bfloat16 and workspace is not None and flash_supported(hd, group):
            runs = _short_and_long(batch, group)
            if runs is not None:
                for run in runs:
                    self._attention_bf16(q, k_pool, v_pool, run, block_table[run.first:run.last], page_size, out, nq, nkv, hd,
                                         window, scale, workspace)
                return
        self._attention_bf16(q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace)

    def _attention_bf16(self, q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace):
        group = nq // nkv
        if (q.dtype == torch.bfloat16 and self.use_tcgen05_attention and getattr(batch, "max_q_len", 0) * group > 16
                and tcgen05_attention_supported(hd, group, page_size)):
            attention_tcgen05(q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace=workspace)
            return
        if q.dtype == torch.bfloat16 and workspace is not None and flash_supported(hd, nq // nkv):
            self.attention_flash(q, k_pool, v_pool, batch, block_table, page_size, out, nq, nkv, hd, window, scale, workspace)
            return
        attention_plain(q, k_pool, v_pool, batch.positions, batch.seq_index, block_table, page_size, out, nq, nkv, hd,
                        window, scale, batch.status)

    def decode_attention_splits(self, n_seqs: int, nkv: int, hd: int, group: int, max_seq_len: int, dtype) -> int:
        """How many blocks share the keys of a (sequence, kv head) when ``n_seqs`` sequences decode one token each:
        the one shape of a decode step's launches that follows the sequences' lengths."""
        # (asked once a layer and step: remembered by what the answer depends on, the length only through its key tiles)
        key = (n_seqs, nkv, hd, group, -(-max_seq_len // 64), dtype)
        found = self._splits_memo.get(key)
        if found is None:
            if len(self._splits_memo) > 4096:
                self._splits_memo.clear()
            found = 1 if dtype != torch.bfloat16 or not flash_supported(hd, group) else flash_splits(n_seqs, nkv, max_seq_len)
            self._splits_memo[key] = found
        return found


# Calls without an engine (tests of single kernels, parts bound by hand) take this one: the fixed rule, no tuning.
default = Kernels("measured")
linear, linear_bf16, attention = default.linear, default.linear_bf16, default.attention
prefers_tcgen05, prefers_fused_swiglu = default.prefers_tcgen05, default.prefers_fused_swiglu
decode_takes_projection = default.decode_takes_projection
