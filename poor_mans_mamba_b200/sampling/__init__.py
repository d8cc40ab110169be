from .sampler import Sampler
