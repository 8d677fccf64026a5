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
            assert lib.vosti_attention_decode_scratch(count, nq, nkv, d, longest) == count * nq * segments * (d + 4)
    # many tokens: one segment per request as long as it fits; few tokens: cut finely
    assert lib.vosti_attention_decode_segment_keys(64, nq, nkv, d, 2560) == 2560
    assert lib.vosti_attention_decode_segment_keys(1, nq, nkv, d, 2560) == 128
    # the choice is a function of the launch's shape, never of a request's place in it
    assert lib.vosti_attention_decode_segment_keys(8, nq, nkv, d, 2560) == lib.vosti_attention_decode_segment_keys(8, nq, nkv, d, 2560)


def test_no_product_is_split_when_one_order_of_arithmetic_is_asked_for(lib):
    assert lib.vosti_fixed_order() == 0
    lib.vosti_set_fixed_order(1)
    try:
        for features, k in [(4096, 4096), (4096, 12288), (151936, 4096), (1000, 1000)]:
            assert {lib.vosti_gemm_tc_splits(t, features, k) for t in (1, 8, 64, 65, 128, 129, 4096)} == {1}
    finally:
        lib.vosti_set_fixed_order(0)
    assert lib.vosti_gemm_tc_splits(8, 4096, 12288) > 1
