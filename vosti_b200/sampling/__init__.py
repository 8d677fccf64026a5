from .sampler import SamplingParams, sample_rows, sampling_arrays, uniform

__all__ = ["SamplingParams", "sample_rows", "sampling_arrays", "uniform"]
