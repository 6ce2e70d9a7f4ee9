"""Random weights from a configuration and a seed.

Every tensor is drawn from its own generator, seeded by (seed, tensor name), so
a tensor's values do not depend on which other tensors exist or in which order
they are made.  Recipes: "linear" and "embedding" N(0, 0.02); "norm"
1 + N(0, 0.05) so that a dropped or misplaced norm weight changes the result
(the reference's fixture has norm weights of exactly 1: scripts/dense_oracle.py:15-20).
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from .safetensors_io import save_file

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def draw(spec, seed: int, device="cpu") -> torch.Tensor:
    """One tensor of ``spec`` in float32 (int32 for integer tables)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(tensor_seed(seed, spec.name))
    shape = tuple(spec.shape)
    if spec.init in ("linear", "embedding"):
        return torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * 0.02
    if spec.init == "norm":
        return 1.0 + torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * 0.05
    if spec.init == "zeros":
        return torch.zeros(shape, device=device, dtype=torch.int32 if spec.keep == "int32" else torch.float32)
    if spec.init == "ones":
        return torch.ones(shape, device=device, dtype=torch.float32)
    raise ValueError(f"unknown init recipe '{spec.init}' for {spec.name}")


def random_tensors(specs: list, seed: int, compute_dtype: torch.dtype, device) -> dict:
    """Tensors for ``specs`` made on ``device`` directly (no folder is written)."""
    from .loader import held_dtype
    out = {}
    for s in specs:
        if s.name not in out:
            t = draw(s, seed, device)
            out[s.name] = t.to(held_dtype(s, t.dtype, compute_dtype))
    return out


def write_random_model(config, folder: str, seed: int = 0, store_dtype: str = "bfloat16") -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed
    configuration of a registered architecture) with random weights."""
    from ..registry import build_model_spec
    if store_dtype not in _STORE:
        raise ValueError(f"store dtype must be one of {sorted(_STORE)}")
    spec = build_model_spec(config)
    os.makedirs(folder, exist_ok=True)
    tensors = {}
    for s in spec.all_param_specs():
        if s.name in tensors:
            continue
        t = draw(s, seed)
        if s.keep == "compute":
            t = t.to(_STORE[store_dtype])
        tensors[s.name] = t
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(config.to_dict(), fh, indent=1)
    save_file(tensors, os.path.join(folder, "model.safetensors"), {"seed": seed, "format": "pt"})
    return folder
