from .sampler import Sampler, pack_sampling

__all__ = ["Sampler", "pack_sampling"]
