"""The launch rules that are functions of sizes only (no GPU needed: the kernel library's host
side answers them): how many K splits a product uses, and how many keys a decode-attention
segment holds. They decide reduction orders, so what they depend on is part of the contract."""
import ctypes

import pytest


@pytest.fixture(scope="module")
def lib():
    try:
        from vosti_b200 import ops
        library = ops.library()
    except Exception as error:                       # no nvcc on this machine
        pytest.skip(f"the kernel library cannot be built here: {error}")
    library.vosti_attention_decode_scratch.restype = ctypes.c_int64
    return library


def test_split_count_depends_on_the_weight_only_up_to_64_tokens(lib):
    for features, k in [(4096, 4096), (6144, 4096), (4096, 12288), (24576, 4096), (151936, 4096), (1000, 1000),
                        (5120, 17408)]:
        counts = {lib.vosti_gemm_tc_splits(t, features, k) for t in (1, 2, 7, 8, 31, 32, 33, 64)}
        assert len(counts) == 1, (features, k, counts)       # a decode batch's size does not change the sum order
        splits = counts.pop()
        tiles, k_blocks = -(-features // 128), -(-k // 64)
        assert 1 <= splits <= 16 and splits * tiles <= max(296, tiles)      # never a second round of CTAs
        assert splits == 1 or k_blocks // splits >= 4
        assert lib.vosti_gemm_tc_splits(129, features, k) == 1 and lib.vosti_gemm_tc_splits(4096, features, k) == 1


def test_decode_segment_length(lib):
    nq, nkv, d = 32, 8, 128
    for count in (1, 2, 8, 31, 64, 256, 1000):
        for longest in (1, 17, 128, 129, 2048, 2560, 4096, 4097, 20000, 131072):
            keys = lib.vosti_attention_decode_segment_keys(count, nq, nkv, d, longest)
            assert 128 <= keys <= 4096 and keys % 64 == 0
            segments = -(-longest // keys)
            assert lib.vosti_attention_decode_scratch(count, nq, nkv, d, longest) >= count * nq * segments * (d + 4)
    # many tokens: one segment per request as long as it fits; few tokens: cut finely
    assert lib.vosti_attention_decode_segment_keys(64, nq, nkv, d, 2560) == 2560
    # one CTA per (token, kv head, segment): the segment count that makes waves x (keys + 350) smallest.
    # While all CTAs fit the GPU at once (296 of them at these sizes) that is as many segments as fit,
    # at most 16 for up to 8 (token, kv head) pairs and 8 beyond, of equal length, a multiple of 64
    assert lib.vosti_attention_decode_segment_keys(1, nq, nkv, d, 2560) == 192        # 8 pairs x 14 segments
    assert lib.vosti_attention_decode_segment_keys(8, nq, nkv, d, 2560) == 640        # 64 pairs x 4
    assert lib.vosti_attention_decode_segment_keys(4, nq, nkv, d, 2560) == 320        # 32 pairs x 8
    assert lib.vosti_attention_decode_segment_keys(16, nq, nkv, d, 2560) == 1280      # 128 pairs x 2
    # in waves: 384 pairs are 2 waves of 2560 keys or 3 of 1280; 512 pairs are 2 waves of 2560 or 4 of 1280
    assert lib.vosti_attention_decode_segment_keys(48, nq, nkv, d, 2560) == 1280
    assert lib.vosti_attention_decode_segment_keys(64, nq, nkv, d, 2560) == 2560
    assert lib.vosti_attention_decode_segment_keys(256, nq, nkv, d, 2560) == 2560
    # too long for 8 segments of 4096 keys: the persistent kernel's cost model
    assert lib.vosti_attention_decode_segment_keys(8, nq, nkv, d, 40000) > 4096 // 2
    assert lib.vosti_set_decode_once(0) == 0
    try:
        # the persistent kernel's cost model alone
        assert lib.vosti_attention_decode_segment_keys(1, nq, nkv, d, 2560) == 128
        assert lib.vosti_attention_decode_segment_keys(64, nq, nkv, d, 2560) == 2560
        for count in (1, 8, 64):
            keys = lib.vosti_attention_decode_segment_keys(count, nq, nkv, d, 2560)
            assert lib.vosti_attention_decode_scratch(count, nq, nkv, d, 2560) == count * nq * -(-2560 // keys) * (d + 4)
    finally:
        assert lib.vosti_set_decode_once(1) == 0
    # a pinned length overrides the cost model for every shape of launch, and taking the pin
    # away gives the launches their own choice back
    shapes = [(c, n) for c in (1, 8, 64) for n in (600, 2560, 9000)]
    free = [lib.vosti_attention_decode_segment_keys(c, nq, nkv, d, n) for c, n in shapes]
    assert len(set(free)) > 1
    assert lib.vosti_set_decode_segment(576) == 0
    try:
        assert {lib.vosti_attention_decode_segment_keys(c, nq, nkv, d, n) for c, n in shapes} == {576}
        assert lib.vosti_set_decode_segment(100) != 0            # not a multiple of 64: refused, the pin stays
        assert lib.vosti_attention_decode_segment_keys(8, nq, nkv, d, 2560) == 576
    finally:
        assert lib.vosti_set_decode_segment(0) == 0
    assert [lib.vosti_attention_decode_segment_keys(c, nq, nkv, d, n) for c, n in shapes] == free


def test_no_product_is_split_when_one_order_of_arithmetic_is_asked_for(lib):
    assert lib.vosti_fixed_order() == 0
    lib.vosti_set_fixed_order(1)
    try:
        for features, k in [(4096, 4096), (4096, 12288), (151936, 4096), (1000, 1000)]:
            assert {lib.vosti_gemm_tc_splits(t, features, k) for t in (1, 8, 64, 65, 128, 129, 4096)} == {1}
    finally:
        lib.vosti_set_fixed_order(0)
    assert lib.vosti_gemm_tc_splits(8, 4096, 12288) > 1


def test_weight_bytes_of_a_decode_step_in_closed_form():
    """What bench.py counts as the weights a decode step must read: every tensor the model
    expects except the embedding table (read by rows), two bytes each. For the 8B sizes that is
    13.892 GB of layers + the final norm + 1.245 GB of output head."""
    import importlib.util
    import math
    import os
    from vosti_b200.config import model_spec_from_config
    from vosti_b200.models import expected_weights
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    spec = importlib.util.spec_from_file_location("bench_for_test", path)
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for size, (_, config) in bench.SIZES.items():
        names = expected_weights(model_spec_from_config(config))
        total = sum(2 * math.prod(w.shape) for name, w in names.items() if name != "model.embed_tokens.weight")
        assert bench.closed_form_weight_bytes(config) == total, size
    layers = bench.closed_form_weight_bytes(bench.SIZES["8b"][1]) - 2 * 151936 * 4096
    assert abs(layers - 13.892e9) < 2e6 and 2 * 151936 * 4096 == 1_244_659_712
