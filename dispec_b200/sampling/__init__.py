from dispec_b200.sampling.sampler import Sampler, SamplingParams, sample

__all__ = ["Sampler", "SamplingParams", "sample"]
