"""A plain, slow implementation of the Qwen3 dense decoder, for tests only.

Whole sequences, no cache, no batching, one function for each part, float64
arithmetic on the CPU.  It shares no code with the engine: it reads the model
folder with the ``safetensors`` package and restates the reference's formulas,
each cited by file:line of d9beuD/rust-mlx.

The reference's own model code cannot be compiled or imported on this machine
(no Rust toolchain, no MLX), so this file rests on the formulas; it is anchored
on the reference's shipped fixture instead (tests/fixtures/dense: weights, a
prompt, the logits of its last position and 32 greedy tokens), see
tests/test_plain_fixture.py and tests/golden/.

``rounding="bfloat16"`` restates what the engine's bfloat16 path stores between
kernels: matrices are rounded to bfloat16, and so is every activation that the
engine writes to memory in bfloat16 (the residual stream, softmax, norms and
rotations stay unrounded, as the engine computes them in 32-bit).
"""
import json
import math
import os

import torch
from safetensors import safe_open

F = torch.float64


def read_folder(folder):
    """config.json as a dict and every tensor by name (src/weights.rs:22-63)."""
    with open(os.path.join(folder, "config.json")) as fh:
        config = json.load(fh)
    tensors = {}
    for name in sorted(os.listdir(folder)):
        if name.endswith(".safetensors"):
            with safe_open(os.path.join(folder, name), framework="pt") as f:
                for key in f.keys():
                    tensors[key] = f.get_tensor(key)
    return config, tensors


def make_round(rounding):
    if rounding in (None, "float32", "none"):
        return lambda t: t
    if rounding == "bfloat16":
        return lambda t: t.to(torch.bfloat16).to(F)
    raise ValueError(rounding)


def rope_theta(config):
    """rope_theta, else rope_parameters.rope_theta, else 1e6 (src/dense.rs:323-332)."""
    if config.get("rope_theta") is not None:
        return float(config["rope_theta"])
    params = config.get("rope_parameters") or {}
    if params.get("rope_theta") is not None:
        return float(params["rope_theta"])
    return 1e6


def layer_windows(config):
    """Window of every layer (0: all keys).  The reference's dense model has no window
    (src/dense.rs:249-256); a window is used only where config.json asks for it."""
    n = config["num_hidden_layers"]
    if not config.get("use_sliding_window"):
        return [0] * n
    w = int(config["sliding_window"])
    kinds = config.get("layer_types")
    if not kinds:
        kinds = ["sliding_attention" if i >= config.get("max_window_layers", 0) else "full_attention"
                 for i in range(n)]
    return [w if k == "sliding_attention" else 0 for k in kinds]


def embedding(table, ids):
    """h = embed_tokens.weight[ids] (src/weights.rs:203-204, src/dense.rs:378-379)."""
    return table[torch.as_tensor(ids, dtype=torch.long, device=table.device)]


def rms_norm(v, weight, eps):
    """v * rsqrt(mean(v^2) + eps) * weight over the last axis (src/dense.rs:382; the
    same shape of formula, written out, in src/compiled.rs:22-28 — dense uses the
    plain weight, not weight + 1)."""
    ms = (v * v).mean(dim=-1, keepdim=True)
    return v * torch.rsqrt(ms + eps) * weight


def linear(x, weight, bias=None, rnd=lambda t: t):
    """y = x . W^T with W stored [out, in] (src/weights.rs:196), plus the bias where the checkpoint has a
    tensor ``<prefix>.bias``: added to the product, which the library has already rounded to the activations'
    dtype (src/weights.rs:96,198-200)."""
    y = rnd(x @ weight.t())
    return y if bias is None else rnd(y + bias)


def rope_frequencies(config, rotary_dim):
    """(inv_freq as float32 [rotary_dim / 2], factor that q and k are each multiplied with).

    Plain: inv_freq[j] = theta^(-2j / rotary_dim), factor 1 (src/dense.rs:187-195: scale 1).  The reference's dense
    model has no scaled variant; "linear" and "yarn" restate the published definitions.  linear: inv_freq / factor.
    yarn: the pair index at which a pair makes b turns within the original context L is
    d(b) = rotary_dim ln(L / (2 pi b)) / (2 ln theta); pairs below floor(d(beta_fast)) keep their frequency, pairs
    above ceil(d(beta_slow)) are divided by factor, linear in the index between; q and k are multiplied by
    0.1 ln(factor) + 1 unless ``attention_factor`` is given."""
    theta = rope_theta(config)
    half = rotary_dim // 2
    inv = theta ** (-2.0 * torch.arange(half, dtype=F) / rotary_dim)
    scaling = config.get("rope_scaling")
    if scaling is None and isinstance(config.get("rope_parameters"), dict) and \
            config["rope_parameters"].get("rope_type", "default") != "default":
        scaling = config["rope_parameters"]
    kind = (scaling or {}).get("rope_type", (scaling or {}).get("type"))
    if kind in (None, "default"):
        return inv.to(torch.float32), 1.0
    factor = float(scaling["factor"])
    if kind == "linear":
        return (inv / factor).to(torch.float32), 1.0
    if kind != "yarn":
        raise ValueError(kind)
    L = float(scaling.get("original_max_position_embeddings") or config["max_position_embeddings"])
    d = lambda b: rotary_dim * math.log(L / (2 * math.pi * b)) / (2 * math.log(theta))  # noqa: E731
    low = max(math.floor(d(scaling.get("beta_fast", 32.0))), 0)
    high = min(math.ceil(d(scaling.get("beta_slow", 1.0))), rotary_dim - 1)
    high = high if high != low else low + 0.001
    out = torch.empty(half, dtype=F)
    for j in range(half):
        share = min(max((j - low) / (high - low), 0.0), 1.0)      # of the divided frequency
        out[j] = share * inv[j] / factor + (1.0 - share) * inv[j]
    given = scaling.get("attention_factor")
    return out.to(torch.float32), float(given) if given is not None else 0.1 * math.log(factor) + 1.0


def rope(x, positions, theta, rotary_dim, inv_freq=None):
    """Half-split rotation of the first ``rotary_dim`` numbers of each head:
    pairs (j, j + rotary_dim/2), inv_freq[j] = theta^(-2j/rotary_dim),
    out[j] = x[j] cos - x[j+half] sin, out[j+half] = x[j+half] cos + x[j] sin
    (src/dense.rs:187-195 with traditional=false; kernels/text_rope.metal:3-14).
    The table of inverse frequencies is held in float32 and the angle is the float32
    product float(pos) * inv_freq[j], as in kernels/text_rope.metal:11 and
    src/rope.rs:21-27; sine, cosine and the rotation are then exact here.
    x: [T, heads, head_dim]; positions: [T]."""
    half = rotary_dim // 2
    j = torch.arange(half, dtype=F, device=x.device)
    if inv_freq is None:
        inv_freq = (theta ** (-2.0 * j / rotary_dim)).to(torch.float32)
    angle = (positions.to(device=x.device, dtype=torch.float32)[:, None] * inv_freq.to(x.device)[None, :]).to(F)   # [T, half]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:rotary_dim]
    out = x.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:rotary_dim] = b * cos + a * sin
    return out


def attention_scores(q, k, v, positions, window, score_factor=1.0):
    """softmax(scale * q k^T + mask) v with scale = head_dim^-0.5, causal mask aligned
    to the end, query head i reading kv head i // (heads / kv_heads)
    (src/dense.rs:221-227, 249-256).  q: [T, nq, hd]; k, v: [T, nkv, hd].
    ``window`` > 0: a query at position p sees keys p - window + 1 .. p only."""
    T, nq, hd = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = hd ** -0.5 * score_factor
    pos = positions.to(device=q.device, dtype=torch.long)
    allowed = pos[None, :] <= pos[:, None]
    if window > 0:
        allowed &= pos[None, :] > pos[:, None] - window
    out = torch.empty_like(q)
    for head in range(nq):
        kh = head // group
        s = (q[:, head, :] @ k[:, kh, :].t()) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, head, :] = p @ v[:, kh, :]
    return out


def attention(x, w, prefix, config, positions, window, rnd, tap=None):
    """q/k/v projections, per-head RMSNorm of q and k before the rotation, rotation of
    all head_dim numbers, attention, output projection (src/dense.rs:139-270)."""
    T = x.shape[0]
    nq, nkv, hd = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    eps = config["rms_norm_eps"]
    b = lambda name: w.get(prefix + name)                                    # noqa: E731  (weights.rs:96)
    q = linear(x, w[prefix + ".q_proj.weight"], b(".q_proj.bias"), rnd).reshape(T, nq, hd)   # dense.rs:147,155
    k = linear(x, w[prefix + ".k_proj.weight"], b(".k_proj.bias"), rnd).reshape(T, nkv, hd)  # dense.rs:157-160
    v = linear(x, w[prefix + ".v_proj.weight"], b(".v_proj.bias"), rnd).reshape(T, nkv, hd)  # dense.rs:161-165
    if tap is not None:
        tap("qkv", torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1))
    q = rms_norm(q, w[prefix + ".q_norm.weight"], eps)                       # dense.rs:169
    k = rms_norm(k, w[prefix + ".k_norm.weight"], eps)                       # dense.rs:175
    theta = rope_theta(config)
    inv_freq, qk_factor = rope_frequencies(config, hd)
    q = rnd(rope(q, positions, theta, hd, inv_freq))                         # dense.rs:187-195
    k = rnd(rope(k, positions, theta, hd, inv_freq))                         # dense.rs:206-214
    o = rnd(attention_scores(q, k, v, positions, window, qk_factor ** 2))    # dense.rs:249-256
    if tap is not None:
        tap("q_rot", q.reshape(T, nq * hd))
        tap("attn_out", o.reshape(T, nq * hd))
    return linear(o.reshape(T, nq * hd), w[prefix + ".o_proj.weight"], b(".o_proj.bias"), rnd)  # dense.rs:258-269


def swiglu_mlp(x, w, prefix, rnd, tap=None):
    """down(silu(gate(x)) * up(x)), silu(z) = z * sigmoid(z) (src/dense.rs:293-298;
    src/compiled.rs:7-12: the product is formed without rounding silu(gate) first)."""
    g = rnd(linear(x, w[prefix + ".gate_proj.weight"]))
    u = rnd(linear(x, w[prefix + ".up_proj.weight"]))
    act = rnd(g * torch.sigmoid(g) * u)
    if tap is not None:
        tap("ffn_act", act)
    return rnd(linear(act, w[prefix + ".down_proj.weight"]))


def prepare_weights(config, tensors, rounding):
    """Weights in float64; for the bfloat16 restatement matrices are rounded to bfloat16
    first, one-dimensional tensors (norm weights) keep the precision they are stored in."""
    out = {}
    for name, t in tensors.items():
        if rounding == "bfloat16" and t.dim() >= 2:
            t = t.to(torch.bfloat16)
        out[name] = t.to(F)
    return out


def forward(config, w, ids, rounding=None, positions=None, intermediates=None):
    """Logits [T, vocab] of the whole sequence ``ids`` (src/dense.rs:371-397).  ``intermediates``: a dictionary
    that receives every layer's named tensors as ``run<i>.<name>`` (the names the reference's trace program
    compares, src/bin/trace.rs:4-24)."""
    rnd = make_round(rounding)
    T = len(ids)
    if any(i < 0 or i >= config["vocab_size"] for i in ids):
        raise ValueError("token outside vocabulary")                          # dense.rs:374-377
    if positions is None:
        positions = torch.arange(T)
    eps = config["rms_norm_eps"]
    windows = layer_windows(config)
    h = embedding(w["model.embed_tokens.weight"], ids)                        # dense.rs:379
    for i in range(config["num_hidden_layers"]):
        p = f"model.layers.{i}"
        tap = None
        if intermediates is not None:
            tap = lambda name, t, i=i: intermediates.__setitem__(f"run{i}.{name}", t.clone())  # noqa: E731
            tap("residual", h)
        x = rnd(rms_norm(h, w[p + ".input_layernorm.weight"], eps))           # dense.rs:382
        a = attention(x, w, p + ".self_attn", config, positions, windows[i], rnd, tap)
        h = h + a                                                             # dense.rs:381
        x2 = rnd(rms_norm(h, w[p + ".post_attention_layernorm.weight"], eps))  # dense.rs:385-389
        m = swiglu_mlp(x2, w, p + ".mlp", rnd, tap)
        h = h + m                                                             # dense.rs:385
        if tap is not None:
            tap("norm1", x), tap("mixer_out", a), tap("norm2", x2), tap("ffn_out", m)
    x = rnd(rms_norm(h, w["model.norm.weight"], eps))                         # dense.rs:391
    head = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings") else w["lm_head.weight"]
    return linear(x, head)                                                    # dense.rs:392-396


def argmax_lowest(logits):
    """Greedy choice; ties go to the lowest id (kernels/greedy_reduce.metal:10-14)."""
    m = logits.max()
    return int(torch.nonzero(logits == m)[0, 0])


def greedy(config, w, prompt, n, rounding=None):
    """n greedy tokens after ``prompt``, recomputing the whole sequence for each
    (the loop of src/bin/parity.rs:41-45 without its cache)."""
    ids = list(prompt)
    out = []
    for _ in range(n):
        t = argmax_lowest(forward(config, w, ids, rounding)[-1])
        out.append(t)
        ids.append(t)
    return out


class PlainModel:
    """A folder read once: ``logits(ids)`` and ``greedy(prompt, n)``."""

    def __init__(self, folder, rounding=None):
        self.config, tensors = read_folder(folder)
        if "head_dim" not in self.config:
            self.config["head_dim"] = self.config["hidden_size"] // self.config["num_attention_heads"]
        self.rounding = rounding
        self.w = prepare_weights(self.config, tensors, rounding)

    def logits(self, ids, intermediates=None):
        return forward(self.config, self.w, list(ids), self.rounding, intermediates=intermediates)

    def greedy(self, prompt, n):
        return greedy(self.config, self.w, prompt, n, self.rounding)
