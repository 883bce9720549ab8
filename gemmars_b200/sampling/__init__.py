from .sampler import BatchSampler, SamplingParams, Xorshift64Star  # noqa: F401
