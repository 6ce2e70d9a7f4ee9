"""A single-GPU inference engine for NVIDIA B200 (sm_100a).

Everything between a request's tokens and its next token: typed configuration
and an architecture registry, safetensors weights, layers put together from
parts, a paged cache manager, one step function over mixed batches, a
scheduler, sampling, and hand-written CUDA kernels.
"""
__version__ = "0.1.0"

from .config import ConfigError, Qwen3Config  # noqa: E402
from .registry import known_architectures, load_config, register_architecture  # noqa: E402


def __getattr__(name):
    # the engine needs torch and the CUDA kernels: it is loaded when first asked for
    if name in ("Engine", "EngineError"):
        from . import engine as _e
        return getattr(_e, name)
    if name == "generate":
        return _generate
    raise AttributeError(name)


def _generate(model, prompt_ids, *, dtype="bfloat16", max_tokens=256, temperature=0.0, seed=0, ignore_eos=False,
              prefill_chunk=128, random_weights=False, cache_tokens=None, page_size=64):
    """Load ``model`` (a folder), generate after each prompt (lists of token ids) and return
    the generated ids.  For repeated use build an ``Engine`` once and call its ``generate``."""
    from .engine import Engine
    need = sum(-(-(len(p) + max_tokens) // page_size) * page_size for p in prompt_ids)
    eng = Engine(model, dtype=dtype, random_weights=random_weights, seed=seed, page_size=page_size,
                 max_tokens=cache_tokens or need, max_requests=max(len(prompt_ids), 1))
    return eng.generate(prompt_ids, max_tokens=max_tokens, temperature=temperature, seed=seed,
                        ignore_eos=ignore_eos, prefill_chunk=prefill_chunk)
