"""Random weights from a configuration and a seed.

Every number is a function of (seed, tensor name, index of the element) alone: a tensor's
values do not depend on which other tensors exist, in which order they are made, or on
which device.  The generator is counter-based and uses integer arithmetic only, so the CPU
and the GPU give the same bits: element i of a tensor takes outputs 3i+1, 3i+2, 3i+3 of a
SplitMix64 stream keyed by a hash of (seed, name), adds their twelve 16-bit pieces (a sum
of twelve uniform numbers: normal to a good approximation, no tails beyond six standard
deviations), and scales the centred integer sum with one float32 multiplication.
Recipes: "linear" and "embedding" N(0, 0.02); "norm" 1 + N(0, 0.05) so that a dropped or
misplaced norm weight changes the result (the reference's fixture has norm weights of
exactly 1: scripts/dense_oracle.py:15-20).
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


def _signed(x: int) -> int:
    """A 64-bit pattern as the int64 that holds it."""
    x &= (1 << 64) - 1
    return x - (1 << 64) if x >> 63 else x


_GOLDEN = _signed(0x9E3779B97F4A7C15)
_MUL1, _MUL2 = _signed(0xBF58476D1CE4E5B9), _signed(0x94D049BB133111EB)
_CHUNK = 1 << 22   # elements made at a time: a dozen int64 temporaries of this size


def _mix(z: torch.Tensor) -> torch.Tensor:
    """SplitMix64's finaliser on int64 tensors (products wrap; shifts are made logical by masking)."""
    z = (z ^ ((z >> 30) & 0x3FFFFFFFF)) * _MUL1
    z = (z ^ ((z >> 27) & 0x1FFFFFFFFF)) * _MUL2
    return z ^ ((z >> 31) & 0x1FFFFFFFF)


def normal(key: int, count: int, std: float, device="cpu") -> torch.Tensor:
    """``count`` float32 numbers of standard deviation ``std``, the same bits on every device."""
    out = torch.empty(count, dtype=torch.float32, device=device)
    # the sum S of twelve uniform integers of 0..65535 has mean 6 * 65535 and variance 65536^2 - 1; 2S - 12 * 65535
    # is an exact integer below 2^24, so its float32 image is exact and one multiplication is the only rounding
    scale = torch.tensor(std / (2.0 * (65536.0 ** 2 - 1.0) ** 0.5), dtype=torch.float32, device=device)
    for start in range(0, count, _CHUNK):
        n = min(_CHUNK, count - start)
        base = torch.arange(start, start + n, dtype=torch.int64, device=device) * 3
        total = torch.zeros(n, dtype=torch.int64, device=device)
        for k in (1, 2, 3):
            h = _mix((base + k) * _GOLDEN + _signed(key))
            for shift in (0, 16, 32, 48):
                total += (h >> shift) & 0xFFFF
        out[start:start + n] = (2 * total - 12 * 65535).to(torch.float32) * scale
    return out


def draw(spec, seed: int, device="cpu") -> torch.Tensor:
    """One tensor of ``spec`` in float32 (int32 for integer tables)."""
    shape = tuple(spec.shape)
    count = 1
    for d in shape:
        count *= int(d)
    if spec.init in ("linear", "embedding"):
        return normal(tensor_seed(seed, spec.name), count, 0.02, device).reshape(shape)
    if spec.init == "norm":
        return (normal(tensor_seed(seed, spec.name), count, 0.05, device) + 1.0).reshape(shape)
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
