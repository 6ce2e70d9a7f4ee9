"""Grouped-query attention over the paged cache.

q, k, v projections -> per-head RMSNorm of q and k (optional) -> rotation of q
and k -> keys and values into the request's pages -> softmax(scale q k^T + causal
mask [+ window]) v -> output projection (src/dense.rs:139-270).  Query head i
reads kv head i // (heads / kv_heads); scale = head_dim^-0.5 unless given.  The
three projections are one matrix product over the concatenated weights
[q; k; v]; each output row is the same dot product as with separate weights.
With ``bias`` the projections take ``<prefix>.bias`` tensors, added to the rounded
product as the reference does (src/weights.rs:96,198-200); the output
projection's is optional in a checkpoint.
"""
from __future__ import annotations

import torch

from .base import CacheSpec, Mixer, ParamSpec


class AttentionMixer(Mixer):
    graph_safe = True

    def __init__(self, prefix: str, width: int, heads: int, kv_heads: int, head_dim: int, position,
                 qk_norm_eps: float | None = None, window: int = 0, scale: float | None = None,
                 bias: bool = False):
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.prefix, self.width = prefix, int(width)
        self.heads, self.kv_heads, self.head_dim = int(heads), int(kv_heads), int(head_dim)
        self.position = position
        self.qk_norm_eps = qk_norm_eps
        self.window = int(window)
        self.scale = (float(scale) if scale is not None else self.head_dim ** -0.5) * float(getattr(position, "score_scale", 1.0))
        self.bias = bool(bias)
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = self.b_qkv = self.b_o = None

    def children(self):
        return [self.position]

    def cache_spec(self):
        return CacheSpec("paged", kv_heads=self.kv_heads, head_dim=self.head_dim, window=self.window)

    def graph_key(self, shape):
        # the one launch shape of a decode step that follows the lengths: into how many blocks the keys are split
        return (self.ctx.ops.decode_attention_splits(shape.n_seqs, self.kv_heads, self.head_dim, self.heads // self.kv_heads,
                                                     shape.max_seq_len, self.ctx.dtype),)

    def param_specs(self):
        p, hd = self.prefix, self.head_dim
        specs = [ParamSpec(f"{p}.q_proj.weight", (self.heads * hd, self.width)),
                 ParamSpec(f"{p}.k_proj.weight", (self.kv_heads * hd, self.width)),
                 ParamSpec(f"{p}.v_proj.weight", (self.kv_heads * hd, self.width)),
                 ParamSpec(f"{p}.o_proj.weight", (self.width, self.heads * hd))]
        if self.qk_norm_eps is not None:
            specs += [ParamSpec(f"{p}.q_norm.weight", (hd,), "norm", "float32"),
                      ParamSpec(f"{p}.k_norm.weight", (hd,), "norm", "float32")]
        if self.bias:
            specs += [ParamSpec(f"{p}.q_proj.bias", (self.heads * hd,), "linear", "float32"),
                      ParamSpec(f"{p}.k_proj.bias", (self.kv_heads * hd,), "linear", "float32"),
                      ParamSpec(f"{p}.v_proj.bias", (self.kv_heads * hd,), "linear", "float32"),
                      ParamSpec(f"{p}.o_proj.bias", (self.width,), "linear", "float32", optional=True)]
        return specs

    def bind(self, tensors, ctx):
        super().bind(tensors, ctx)
        p = self.prefix
        self.w_qkv = torch.cat([tensors.pop(f"{p}.q_proj.weight"), tensors.pop(f"{p}.k_proj.weight"),
                                tensors.pop(f"{p}.v_proj.weight")], dim=0).contiguous()
        self.w_o = tensors[f"{p}.o_proj.weight"].contiguous()
        if self.qk_norm_eps is not None:
            self.q_norm = tensors[f"{p}.q_norm.weight"].contiguous()
            self.k_norm = tensors[f"{p}.k_norm.weight"].contiguous()
        if self.bias:
            self.b_qkv = torch.cat([tensors.pop(f"{p}.q_proj.bias"), tensors.pop(f"{p}.k_proj.bias"),
                                    tensors.pop(f"{p}.v_proj.bias")]).contiguous()
            self.b_o = tensors.get(f"{p}.o_proj.bias")

    def linear_weights(self):
        return [self.w_qkv, self.w_o]

    def forward(self, x, batch, cache):
        ops, ws, dt = self.ctx.ops, self.ctx.workspace, self.ctx.dtype
        n = x.shape[0]
        nq, nkv, hd = self.heads, self.kv_heads, self.head_dim
        q = ws.get("q_rot", (n, nq * hd), dt)
        angles = self.position.angles(batch)
        projection = None
        qkv = ws.get("qkv", (n, (nq + 2 * nkv) * hd), dt)
        ops.linear(x, self.w_qkv, qkv, ws, batch.status)
        if self.b_qkv is not None:
            ops.add_bias(qkv, self.b_qkv)
        tap = self.ctx.tap
        if tap is not None:
            tap("qkv", qkv)
        if ops.decode_takes_projection(batch, dt, hd, nq // nkv, cache.page_size, self.position.rotary_dim, angles):
            # decoding: the attention kernel norms, rotates and stores its own token while it waits for its keys
            projection = (qkv, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, angles, not cache.read_only)
        else:
            ops.qk_rope_cache(qkv, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, self.position.inv_freq,
                              self.position.rotary_dim, batch.positions, batch.seq_index, cache.block_table,
                              cache.page_size, cache.k_pool, cache.v_pool, q, nq, nkv, hd, not cache.read_only,
                              batch.status, angles)
        if tap is not None and projection is None:
            tap("q_rot", q)
        o = ws.get("attn_out", (n, nq * hd), dt)
        ops.attention(q, cache.k_pool, cache.v_pool, batch, cache.block_table, cache.page_size, o, nq, nkv, hd,
                      cache.window, self.scale, ws, projection=projection)
        if tap is not None:
            tap("attn_out", o)
        y = ws.get("mixer_out", (n, self.width), dt)
        ops.linear(o, self.w_o, y, ws, batch.status)
        if self.b_o is not None:
            ops.add_bias(y, self.b_o)
        return y
