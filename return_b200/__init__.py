"""return_b200: a one-GPU inference engine for the Qwen3 dense decoder on B200 (sm_100a).

Everything between a request's tokens and its next token: typed configuration and an
architecture registry, safetensors weights by name, layers put together from parts, a paged
cache with block tables and state slots, one step function over mixed batches, a scheduler,
sampling, and hand-written CUDA kernels.  After the rollout engine of wenhaoli-xmu/ReTurn.
"""
from . import parts  # noqa: F401  registers the built-in parts
from .config import registry  # noqa: F401  registers the built-in architecture

__version__ = "0.1.0"
