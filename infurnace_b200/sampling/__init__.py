from .sampler import Sampler, uniform  # noqa: F401
