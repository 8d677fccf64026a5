"""Helpers for GPU tests that drive parts and toy models without the scheduler."""
import torch

from vosti_b200.cache import CacheManager
from vosti_b200.engine.batch import StagingBuffer, StepEntry, build_context


class Harness:
    """A cache manager plus what is needed to build a step's context for given entries."""

    def __init__(self, cache_specs, state_specs, dtype, num_pages=64, page_size=8, max_requests=4):
        self.device = torch.device("cuda:0")
        self.dtype = dtype
        self.cache = CacheManager(cache_specs, state_specs, num_pages=num_pages, page_size=page_size,
                                  max_requests=max_requests, device=self.device, dtype=dtype, prefix_reuse=False)
        self.staging = StagingBuffer(self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)

    def context(self, entries):
        for e in entries:
            if e.request_id not in self.cache.live:
                self.cache.begin(e.request_id)
        return build_context(self.staging, self.cache, entries, self.status, self.dtype)
