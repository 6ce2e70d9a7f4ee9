"""Configuration of the Qwen3 dense decoder.

Keys follow the reference's ``DenseConfig`` (src/dense.rs:12-25): model_type,
hidden_size, num_hidden_layers, num_attention_heads, num_key_value_heads,
head_dim, rms_norm_eps, rope_theta (or rope_parameters.rope_theta, else 1e6:
src/dense.rs:323-332), tie_word_embeddings, vocab_size.  The reference takes the
feed-forward width from the tensors; here ``intermediate_size`` is read so that
shapes can be checked before loading.  ``eos_token_id`` (an integer or a list) is
what the command line stops at (src/bin/infer.rs:102-106).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .base import ModelConfig


@dataclass
class Qwen3Config(ModelConfig):
    hidden_size: int = None  # type: ignore[assignment]
    intermediate_size: int = None  # type: ignore[assignment]
    num_hidden_layers: int = None  # type: ignore[assignment]
    num_attention_heads: int = None  # type: ignore[assignment]
    num_key_value_heads: int = None  # type: ignore[assignment]
    vocab_size: int = None  # type: ignore[assignment]
    rms_norm_eps: float = None  # type: ignore[assignment]
    head_dim: int = 0  # 0: hidden_size // num_attention_heads
    rope_theta: float = 1e6
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    max_position_embeddings: int = 0  # 0: not stated; informational
    use_sliding_window: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0
    layer_types: tuple = ()
    eos_token_id: tuple = ()
    rope_scaling: Optional[dict] = None

    _aliases = {"rope_theta": ("rope_parameters.rope_theta",)}
    _required = ("model_type", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                 "num_key_value_heads", "vocab_size", "rms_norm_eps")

    def validate(self) -> list:
        p = []
        if self.model_type != "qwen3":
            p.append(f"model_type is '{self.model_type}', this configuration reads 'qwen3'")
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "vocab_size"):
            if getattr(self, name) is None or getattr(self, name) <= 0:
                p.append(f"{name} must be positive")
        if p:
            return p
        if self.head_dim == 0:
            if self.hidden_size % self.num_attention_heads:
                p.append("head_dim is absent and hidden_size is not a multiple of num_attention_heads")
            else:
                self.head_dim = self.hidden_size // self.num_attention_heads
        if self.head_dim < 0 or self.head_dim % 2:
            p.append(f"head_dim {self.head_dim} must be a positive even number (rotation works on pairs)")
        if self.num_attention_heads % self.num_key_value_heads:
            p.append("num_attention_heads must be a multiple of num_key_value_heads")
        if not (self.rms_norm_eps > 0):
            p.append("rms_norm_eps must be positive")
        if not (self.rope_theta > 0):
            p.append("rope_theta must be positive")
        scaling = self.rope_scaling_parameters()
        if scaling is not None:
            kind = scaling.get("rope_type", scaling.get("type"))
            if kind not in (None, "default", "linear", "yarn"):
                p.append(f"rope_scaling of type '{kind}' is not supported (default, linear, yarn)")
            elif kind in ("linear", "yarn"):
                factor = scaling.get("factor")
                if isinstance(factor, bool) or not isinstance(factor, (int, float)) or factor < 1:
                    p.append("rope_scaling needs a factor of at least 1")
                if kind == "yarn" and not (scaling.get("original_max_position_embeddings") or 0) > 0:
                    p.append("rope_scaling of type 'yarn' needs original_max_position_embeddings")
        if self.use_sliding_window:
            if self.sliding_window <= 0:
                p.append("use_sliding_window is true but sliding_window is not a positive number")
            if self.layer_types:
                if len(self.layer_types) != self.num_hidden_layers:
                    p.append("layer_types must name every layer")
                bad = sorted({t for t in self.layer_types if t not in ("full_attention", "sliding_attention")})
                if bad:
                    p.append(f"unknown layer_types {bad}")
        return p

    def rope_scaling_parameters(self):
        """The dictionary that scales the rotation, or None: ``rope_scaling``, else ``rope_parameters`` when that
        names a ``rope_type`` (newer checkpoints keep theta and the scaling together there).  A yarn dictionary
        without ``original_max_position_embeddings`` takes the configuration's ``max_position_embeddings``."""
        found = self.rope_scaling
        if found is None:
            params = (getattr(self, "_raw", None) or {}).get("rope_parameters")
            if isinstance(params, dict) and params.get("rope_type", params.get("type")) not in (None, "default"):
                found = params
        if found is None:
            return None
        found = dict(found)
        if found.get("rope_type", found.get("type")) == "yarn" and not found.get("original_max_position_embeddings"):
            found["original_max_position_embeddings"] = self.max_position_embeddings
        return found

    def attention_kinds(self) -> tuple:
        """The mixer of every layer: 'full_attention' or 'sliding_attention'.

        Without ``use_sliding_window`` every layer attends to all keys, which is the
        only case the reference's dense model has (src/dense.rs:249-256).  With it,
        ``layer_types`` decides, or else layers from ``max_window_layers`` on slide.
        """
        n = self.num_hidden_layers
        if not self.use_sliding_window:
            return ("full_attention",) * n
        if self.layer_types:
            return tuple(self.layer_types)
        return tuple("sliding_attention" if i >= self.max_window_layers else "full_attention" for i in range(n))

    def to_dict(self) -> dict:
        out = super().to_dict()
        if self.rope_scaling is None:
            out.pop("rope_scaling")
        if not self.use_sliding_window:
            for k in ("sliding_window", "max_window_layers", "layer_types"):
                out.pop(k)
        if not self.eos_token_id:
            out.pop("eos_token_id")
        if not self.max_position_embeddings:
            out.pop("max_position_embeddings")
        if not out.get("architectures"):
            out["architectures"] = ["Qwen3ForCausalLM"]
        return out
