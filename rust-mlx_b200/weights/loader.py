"""Loading a model's tensors by name.

The model says which tensors it needs (``ParamSpec``: name, shape, how it is
kept); the loader finds them in the folder's safetensors files, checks names and
shapes, and puts them on the device.  Unlike the reference, which reports the
first missing tensor when it is asked for (src/weights.rs:64-69) and stops at a
duplicate (56-59), every problem of a folder is collected into one error.

How a tensor is kept: floating tensors with ``keep == "compute"`` take the run's
dtype (bfloat16, or float32 for the 32-bit path; bfloat16 -> float32 is exact,
float32 -> bfloat16 rounds to nearest even); ``keep == "float32"`` stays 32-bit
in every run; ``keep == "int32"`` tables are held as int32.
"""
from __future__ import annotations

import fnmatch

import torch

from .safetensors_io import SafetensorsError, open_model_files


class WeightsError(ValueError):
    """The folder's tensors do not fit the model; the message lists every problem."""

    def __init__(self, folder, missing=(), unexpected=(), wrong=(), duplicate=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong = list(wrong)
        self.duplicate = list(duplicate)
        lines = [f"weights in {folder} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shape or dtype ({len(self.wrong)}): " + "; ".join(self.wrong))
        if self.duplicate:
            lines.append(f"  present in more than one file ({len(self.duplicate)}): " + ", ".join(self.duplicate))
        super().__init__("\n".join(lines))


def index_folder(folder: str) -> tuple:
    """Open every safetensors file of ``folder``: (name -> TensorEntry, duplicated names)."""
    entries, duplicate = {}, []
    for f in open_model_files(folder):
        for name, e in f.entries.items():
            if name in entries:
                duplicate.append(name)
            entries[name] = e
    return entries, duplicate


def check_tensors(folder: str, entries: dict, duplicate: list, specs: list, ignore: tuple = ()) -> None:
    want = {}
    for s in specs:
        want[s.name] = s
    missing = [n for n in want if n not in entries and not want[n].optional]
    unexpected = [n for n in entries if n not in want and not any(fnmatch.fnmatch(n, pat) for pat in ignore)]
    wrong = []
    for name, s in want.items():
        e = entries.get(name)
        if e is None:
            continue
        if tuple(e.shape) != tuple(s.shape):
            wrong.append(f"{name} has shape {list(e.shape)}, the model needs {list(s.shape)}")
        elif s.keep == "int32" and e.dtype.is_floating_point:
            wrong.append(f"{name} is stored as {e.dtype}, the model needs an integer table")
        elif s.keep != "int32" and not e.dtype.is_floating_point:
            wrong.append(f"{name} is stored as {e.dtype}, the model needs floating point")
    if missing or unexpected or wrong or duplicate:
        raise WeightsError(folder, sorted(missing), sorted(unexpected), wrong, sorted(duplicate))


def held_dtype(spec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if spec.keep == "int32":
        return torch.int32
    if spec.keep == "float32":
        return torch.float32
    return compute


def load_tensors(folder: str, specs: list, compute_dtype: torch.dtype, device, ignore: tuple = (),
                 progress=None) -> dict:
    """Check the folder against ``specs`` and return name -> tensor on ``device``."""
    try:
        entries, duplicate = index_folder(folder)
    except (SafetensorsError, FileNotFoundError) as e:
        raise WeightsError(folder, wrong=[str(e)]) from None
    check_tensors(folder, entries, duplicate, specs, ignore)
    out = {}
    for i, s in enumerate(specs):
        if s.name in out or (s.optional and s.name not in entries):
            continue
        t = entries[s.name].load()
        out[s.name] = t.to(device=device, dtype=held_dtype(s, t.dtype, compute_dtype))
        if progress is not None:
            progress(i + 1, len(specs), s.name)
    return out
