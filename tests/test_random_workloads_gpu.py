"""Randomized workloads through the engine against a roomy, plain engine of the same model:
random prompts (half of them sharing a prefix), arrival steps, page sizes (8 to 64), pool sizes
down to what one request needs (so that requests are preempted and published pages evicted),
row and token limits, portions, prefix reuse, CUDA graphs and async scheduling on or off, greedy
or temperature sampling. float32 must give the same tokens; so must bfloat16 with one order of
arithmetic (`batch_invariant="full"`), where any changed bit of a logit would soon change a
sampled token."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", range(4))
def test_random_workloads_give_the_tokens_of_a_roomy_engine(seed, model_dirs):
    from vosti_b200 import Engine, ops
    try:
        for r in range(12):
            rng = random.Random(seed * 1000 + r)
            name = rng.choice("abc")
            path, config, _ = model_dirs[name]
            limit = config["max_position_embeddings"]
            dtype, mode = rng.choice([("float32", False), ("bfloat16", "full")])
            n = rng.randint(2, 7)
            gen = torch.Generator().manual_seed(seed * 100 + r)
            shared = torch.randint(0, config["vocab_size"], (rng.randint(8, 40),), generator=gen).tolist()
            prompts = []
            for _ in range(n):
                p = torch.randint(0, config["vocab_size"], (rng.randint(1, min(90, limit - 40)),), generator=gen).tolist()
                prompts.append((shared + p)[:limit - 40] if rng.random() < 0.5 else p)
            new_tokens = rng.randint(1, 30)
            temperature = rng.choice([0.0, 0.8])
            seeds = [rng.randint(0, 2 ** 40) for _ in range(n)]
            roomy = Engine(path, dtype=dtype, num_blocks=512, block_size=16, max_num_seqs=8, enable_prefix_caching=False,
                           cuda_graphs=False, batch_invariant=mode)
            want = roomy.generate(prompts, max_tokens=new_tokens, temperature=temperature, seeds=seeds)
            page = rng.choice([8, 16, 32, 48, 64])
            need = max(-(-(len(p) + new_tokens) // page) for p in prompts)
            settings = dict(num_blocks=rng.choice([need, need + 2, 3 * need, 64]), block_size=page,
                            max_num_seqs=rng.choice([1, 2, 3, 8]),
                            max_num_batched_tokens=max(page, rng.choice([page, 2 * page, 64, 256])),
                            prefill_chunk_size=rng.choice([0, page, 2 * page]), enable_prefix_caching=rng.random() < 0.6,
                            cuda_graphs=rng.random() < 0.7, async_scheduling=rng.random() < 0.6, batch_invariant=mode)
            engine = Engine(path, dtype=dtype, **settings)
            got = engine.generate(prompts, max_tokens=new_tokens, temperature=temperature, seeds=seeds,
                                  arrival_steps=sorted(rng.randint(0, 25) for _ in range(n)))
            engine.runner.cache.check()
            assert got == want, (name, dtype, settings, temperature, [len(p) for p in prompts])
            assert engine.runner.cache.available_pages() == settings["num_blocks"] or settings["enable_prefix_caching"]
    finally:
        ops.set_invariance("off")
