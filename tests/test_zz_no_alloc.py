"""The library's entry point that allocates nothing (vosti_b200/csrc/no_alloc.h).

Some users of the kernel library cannot allocate device memory when they call it: a
serving process that gave all free GPU memory to its cache pool at start-up, or a host whose
device memory belongs to another allocator. For them `vosti_gemm_tc_split_static` keeps the
split-K partial sums in a device array inside the library instead of a workspace the caller
allocates. This test calls it through its exported C symbol, twice in a row with different
sizes and data (one for each width of token tile the kernel has), and checks each result
against the ordinary entry point; it also checks that sizes beyond the array are refused and
that, after the warm-up call the header asks for, a call leaves the free device memory as it
found it. It runs last (file name) so that a run that stops at the
first failure has already run every other test, and it passes alone in a fresh process too.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from vosti_b200.csrc import build
    lib = ctypes.CDLL(str(build.library_path()))
    lib.vosti_last_error.restype = ctypes.c_char_p
    return lib


def _static_product(lib, x, w, out_dtype):
    y = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
    status = torch.zeros(1, dtype=torch.int32, device=x.device)
    rc = lib.vosti_gemm_tc_split_static(
        ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(y.data_ptr()),
        x.shape[0], w.shape[0], x.shape[1], int(out_dtype == torch.float32), ctypes.c_void_p(status.data_ptr()),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.vosti_last_error().decode()
    assert status.item() == 0
    return y


def test_static_scratch_product_matches_the_ordinary_entry_point():
    from vosti_b200 import ops
    device = torch.device("cuda:0")
    ops.require_device(device)
    lib = _library()
    status = torch.zeros(1, dtype=torch.int32, device=device)
    torch.manual_seed(0)
    # two calls in a row: the second reuses the array the first one filled
    for tokens, features, k, out_dtype in [(8, 4096, 4096, torch.bfloat16), (70, 1024, 12288, torch.float32),
                                           (1, 6144, 4096, torch.bfloat16), (40, 2048, 8192, torch.bfloat16),
                                           (64, 1536, 4096, torch.float32)]:
        assert lib.vosti_gemm_tc_splits(tokens, features, k) > 1           # the scratch is really used
        x = torch.randn(tokens, k, device=device).bfloat16()
        w = (torch.randn(features, k, device=device) / math.sqrt(k)).bfloat16()
        got = _static_product(lib, x, w, out_dtype)
        want = ops.gemm_tc(x, w, status, out_dtype=out_dtype)
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        assert torch.equal(got, want)                                       # same kernels, same order of sums
        exact = x.double() @ w.double().T
        assert torch.allclose(got.double(), exact, atol=2e-2, rtol=2e-2)
    torch.cuda.synchronize()


def test_static_scratch_calls_leave_device_memory_alone():
    """After one warm-up call on the device, calls neither take nor give back device memory:
    the driver's count of free bytes and torch's own count of what it holds stay the same
    across them (inputs and outputs are made before the counts are read)."""
    from vosti_b200 import ops
    device = torch.device("cuda:0")
    ops.require_device(device)
    lib = _library()
    cases = []
    for tokens, features, k in [(8, 4096, 4096), (48, 1024, 8192), (100, 1024, 4096)]:
        x = torch.randn(tokens, k, device=device).bfloat16()
        w = (torch.randn(features, k, device=device) / math.sqrt(k)).bfloat16()
        y = torch.empty((tokens, features), dtype=torch.bfloat16, device=device)
        cases.append((x, w, y))
    status = torch.zeros(1, dtype=torch.int32, device=device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(x, w, y):
        return lib.vosti_gemm_tc_split_static(
            ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(y.data_ptr()),
            x.shape[0], w.shape[0], x.shape[1], 0, ctypes.c_void_p(status.data_ptr()), stream)

    for case in cases:                     # the warm-up calls: every tile width's kernel is loaded and set up
        assert call(*case) == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(device)
    held_before = torch.cuda.memory_reserved(device)
    for _ in range(3):
        for case in cases:
            assert call(*case) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(device)
    assert free_after == free_before and torch.cuda.memory_reserved(device) == held_before
    assert status.item() == 0


def test_static_scratch_refuses_sizes_beyond_the_array():
    lib = _library()
    device = torch.device("cuda:0")
    x = torch.zeros(129, 4096, device=device).bfloat16()
    w = torch.zeros(8192, 4096, device=device).bfloat16()
    y = torch.empty(129, 8192, device=device).bfloat16()
    args = lambda tokens: (ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(y.data_ptr()),
                           tokens, 8192, 4096, 0, None, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    splits = lib.vosti_gemm_tc_splits(128, 8192, 4096)
    assert splits > 1 and splits * 128 * 8192 > 2 * 1024 * 1024          # more than the array holds
    assert lib.vosti_gemm_tc_split_static(*args(128)) == -1
    assert b"scratch floats" in lib.vosti_last_error()
    assert lib.vosti_gemm_tc_split_static(*args(129)) == -1
    assert b"tokens must be 1..128" in lib.vosti_last_error()
    assert lib.vosti_gemm_tc_split_static(*args(0)) == -1
    assert lib.vosti_gemm_tc_split_static(*args(16)) == 0                 # and a size that fits is served
    torch.cuda.synchronize()
