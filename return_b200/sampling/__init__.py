from .sampler import Sampler, uniform_draw  # noqa: F401
