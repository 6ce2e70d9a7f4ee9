"""A single-GPU inference engine for NVIDIA B200 (sm_100a).

Everything between a request's tokens and its next token: typed configuration
and an architecture registry, safetensors weights, layers put together from
parts, a paged cache manager, one step function over mixed batches, a
scheduler, sampling, and hand-written CUDA kernels.
"""
__version__ = "0.1.0"
