"""The allocation-free decode-attention entry point, called through its exported C
symbol, against the ordinary entry point.

Some embedders may not call cudaMalloc at all (a fixed memory map, another framework's
pool, an open stream capture elsewhere in the process); for them the library carries the
kernel's scratch inside its own image.  This file is named so that pytest collects it
last: a run that stops at the first failure has then already run every other test.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

HEAD_DIM, NQ, NKV, PAGE = 64, 8, 2, 16
ERR_TOO_LARGE = 10010


def _library():
    from llm_runtime_study_b200.csrc.build import load_library
    from llm_runtime_study_b200.ops import attention_bf16, native

    name = attention_bf16.library_name(HEAD_DIM)
    lib = load_library(name, ("attention_mma.cu",), native.library_defines(name))
    fn = lib.b200_attention_decode_bf16_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return fn


def _case(seed, lens):
    g = torch.Generator().manual_seed(seed)
    pages_per = -(-max(lens) // PAGE)
    total = pages_per * len(lens)
    order = torch.randperm(total, generator=g).to(torch.int32).view(len(lens), pages_per)
    keys = torch.randn(total, NKV, PAGE, HEAD_DIM, generator=g).bfloat16().cuda()
    values = torch.randn(total, NKV, PAGE, HEAD_DIM, generator=g).bfloat16().cuda()
    q = torch.randn(len(lens), NQ, HEAD_DIM, generator=g).bfloat16().cuda()
    return q, keys, values, torch.tensor(lens, dtype=torch.int32).cuda(), order.cuda()


def _call(fn, q, keys, values, kv_len, table, splits):
    out = torch.empty_like(q)
    status = fn(q.data_ptr(), keys.data_ptr(), values.data_ptr(), out.data_ptr(), kv_len.data_ptr(), table.data_ptr(),
                table.shape[1], PAGE, q.shape[0], NQ, NKV, 1 / math.sqrt(HEAD_DIM), 0, splits,
                torch.cuda.current_stream().cuda_stream)
    return status, out


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    from llm_runtime_study_b200.ops import attention_bf16

    fn = _library()
    # the second call has other inputs and another split count: what the first left in the
    # shared scratch must not matter
    for seed, lens, splits in ((1, [700, 33, 64, 129, 1], 5), (2, [95, 300], 3)):
        q, keys, values, kv_len, table = _case(seed, lens)
        want = attention_bf16.decode_attention(q, keys, values, kv_len=kv_len, block_table=table,
                                               scale=1 / math.sqrt(HEAD_DIM), splits=splits, backend="mma")
        status, got = _call(fn, q, keys, values, kv_len, table, splits)
        assert status == 0
        torch.cuda.synchronize()
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        assert torch.equal(got, want)      # same kernels, same order of sums


def test_a_warmed_call_takes_no_device_memory():
    """What the entry point is for: after its first call on the device (which looks up the address of the
    scratch array) a call neither takes nor gives back device memory.  Seen from outside: the driver's count
    of free memory is the same before and after, and so is the count of torch's allocator, which the test's
    own tensors come from."""

    fn = _library()
    q, keys, values, kv_len, table = _case(4, [500, 130, 64])
    out = torch.empty_like(q)
    args = (q.data_ptr(), keys.data_ptr(), values.data_ptr(), out.data_ptr(), kv_len.data_ptr(), table.data_ptr(),
            table.shape[1], PAGE, q.shape[0], NQ, NKV, 1 / math.sqrt(HEAD_DIM), 0, 4, torch.cuda.current_stream().cuda_stream)
    assert fn(*args) == 0                                      # the first call on this device sets up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    for _ in range(3):
        assert fn(*args) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before and torch.cuda.memory_reserved() == reserved_before


def test_refuses_what_does_not_fit_and_launches_nothing():
    fn = _library()
    q, keys, values, kv_len, table = _case(3, [64] * 4)
    big_q = torch.zeros(2048, NQ, HEAD_DIM, dtype=torch.bfloat16, device="cuda")     # 2048 * 8 * 16 * 66 floats > 1 Mi
    out = torch.full_like(big_q, 7.0)
    status = fn(big_q.data_ptr(), keys.data_ptr(), values.data_ptr(), out.data_ptr(), kv_len.data_ptr(), table.data_ptr(),
                table.shape[1], PAGE, 2048, NQ, NKV, 0.125, 0, 16, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status == ERR_TOO_LARGE
    assert float(out.float().min()) == 7.0
    status, _ = _call(fn, q, keys, values, kv_len, table, 1)                          # one part needs no scratch
    assert status == 0
