from .sampler import (SamplingParams, sample_from_slots, sample_rows, sampler_state_words, sampling_arrays,
                      uniform)

__all__ = ["SamplingParams", "sample_from_slots", "sample_rows", "sampler_state_words", "sampling_arrays", "uniform"]
